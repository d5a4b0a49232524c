"""Op registration in the `xma::` namespace, as xma/custom_op.py:64-90 does it: out-parameter style
functions that return None, registered with torch.library.custom_op and `mutates_args`, so that
torch.compile(fullgraph=True) can functionalise them."""

from __future__ import annotations

import inspect
from typing import Callable, Iterable, Sequence

import torch

LIBRARY_NAME = "xma"


def ctx_needs_gradients(ctx) -> bool:
    return any(ctx.needs_input_grad)


def ctx_save_for_backward(ctx, *args) -> None:
    if ctx_needs_gradients(ctx):
        ctx.save_for_backward(*args)


def xma_op(
    mutates_args: str | Iterable[str] = None,
    device_types: str | Sequence[str] | None = None,
    schema: str | None = None,
    fake_func: Callable | None = None,
) -> Callable:
    def _inner(func: Callable):
        custom_op = torch.library.custom_op(
            f"{LIBRARY_NAME}::{func.__name__}", func, mutates_args=mutates_args, device_types=device_types, schema=schema
        )
        if fake_func is not None:
            custom_op.register_fake(fake_func)

        def _run(*args, **kwargs):
            # Under torch.compile the registered op is what the graph records; in eager mode the body
            # is called directly, which skips the dispatcher's per-call bookkeeping (tens of
            # microseconds per launch, visible next to sub-millisecond kernels).
            if torch.compiler.is_compiling():
                return custom_op(*args, **kwargs)
            return func(*args, **kwargs)

        _run.__signature__ = inspect.signature(func)
        _run.__name__ = func.__name__
        return _run

    return _inner
