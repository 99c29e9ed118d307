"""Optional one-line report of every op call's operand sizes.

Same switches and line prefix as the reference's ``deepgemm/print_size.py`` (:8-10, :97-99,
:432-457): set ``DEEPGEMM_PRINT_OP_SIZE=1`` before importing the package and every call of a
``deepgemm.op`` entry point prints ``[DeepGEMM][size] <op> name=(shape):dtype:device ...
E= M= N= K=``; ``DEEPGEMM_PRINT_OP_SIZE_FILTER=a,b`` keeps only ops whose name contains one of
the substrings; ``DEEPGEMM_PRINT_OP_SIZE_STATS=1`` adds sum / min / max of ``masked_m`` (that
one reads the tensor back, so it synchronises).  Unlike the reference, which keeps one
formatter per op, the fields here come from the wrapped function's own signature.
"""
from __future__ import annotations

import functools
import inspect
import os
from typing import Any, Callable, List

_ENV_ENABLE = "DEEPGEMM_PRINT_OP_SIZE"
_ENV_STATS = "DEEPGEMM_PRINT_OP_SIZE_STATS"
_ENV_FILTER = "DEEPGEMM_PRINT_OP_SIZE_FILTER"
_WRAPPED = "__deepgemm_print_size_wrapped__"


def _flag(name: str) -> bool:
    return os.environ.get(name, "0") not in ("", "0", "false", "False")


PRINT_SIZE_ENABLED = _flag(_ENV_ENABLE)


def describe(x: Any) -> str:
    """``(d0,d1,...):dtype:device`` for tensors, ``str(x)`` for anything else."""
    if x is None:
        return "None"
    shape = getattr(x, "shape", None)
    if shape is None:
        return str(x)
    text = "(" + ",".join(str(int(v)) for v in shape) + ")"
    if getattr(x, "dtype", None) is not None:
        text += ":" + str(x.dtype).replace("torch.", "")
    if getattr(x, "device", None) is not None:
        text += ":" + str(x.device)
    return text


def _wanted(op_name: str) -> bool:
    needles = [s.strip() for s in os.environ.get(_ENV_FILTER, "").split(",") if s.strip()]
    return not needles or any(n in op_name for n in needles)


def _problem_dims(bound: dict) -> List[str]:
    """E / M / N / K as the reference prints them: from the activation, weight and output."""
    act = next((bound[k] for k in ("input", "matrix_a") if k in bound), None)
    wgt = next((bound[k] for k in ("b_qweight", "matrix_b") if k in bound), None)
    out = next((bound[k] for k in ("output", "matrix_c") if k in bound), None)
    if act is None or out is None or getattr(act, "dim", None) is None:
        return []
    masked = act.dim() == 3
    experts = act.shape[0] if masked else (wgt.shape[0] if wgt is not None else 0)
    return [f"E={int(experts)}", f"M={int(act.shape[1] if masked else act.shape[0])}",
            f"N={int(out.shape[-1])}", f"K={int(act.shape[-1])}"]


def _count_stats(bound: dict) -> List[str]:
    if not _flag(_ENV_STATS):
        return []
    for key in ("masked_m", "actual_tokens", "token_per_expert"):
        t = bound.get(key)
        if t is not None and hasattr(t, "sum"):
            return [f"{key}_sum={int(t.sum())}", f"{key}_min={int(t.min())}", f"{key}_max={int(t.max())}"]
    return []


def format_call(fn: Callable[..., Any], *args: Any, **kwargs: Any) -> List[str]:
    bound = inspect.signature(fn).bind_partial(*args, **kwargs).arguments
    fields = [f"{name}={describe(value)}" for name, value in bound.items()]
    return fields + _problem_dims(bound) + _count_stats(bound)


def wrap(op_name: str, fn: Callable[..., Any]) -> Callable[..., Any]:
    if getattr(fn, _WRAPPED, False):
        return fn

    @functools.wraps(fn)
    def wrapped(*args: Any, **kwargs: Any) -> Any:
        if _wanted(op_name):
            try:
                print("[DeepGEMM][size]", op_name, *format_call(fn, *args, **kwargs))
            except Exception as exc:  # the report must never break the call
                print("[DeepGEMM][size]", op_name, f"format_error={type(exc).__name__}")
        return fn(*args, **kwargs)

    setattr(wrapped, _WRAPPED, True)
    return wrapped


def install_op_size_printer(op_module: Any, force: bool = False) -> None:
    """Wraps every public function of ``op_module`` (normally ``deepgemm.op``).  Does nothing
    unless ``DEEPGEMM_PRINT_OP_SIZE`` was set at import time or ``force`` is given."""
    if not (PRINT_SIZE_ENABLED or force):
        return
    for name, fn in list(vars(op_module).items()):
        if name.startswith("_") or not inspect.isfunction(fn) or fn.__module__ != op_module.__name__:
            continue
        setattr(op_module, name, wrap(name, fn))
