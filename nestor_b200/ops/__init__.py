"""Hot-op entry points.

Every op has two bodies: the PyTorch statement in :mod:`nestor_b200.ops.reference` (CPU
execution and test oracle) and the sm_100a kernels behind :mod:`nestor_b200.ops.cuda`.
CUDA tensors take the kernel body; if the compiled extension is missing on a CUDA
machine the import fails loudly instead of silently running PyTorch ops.
``NESTOR_B200_REFERENCE_OPS=1`` forces the oracle on CUDA tensors (debugging only).
"""

from __future__ import annotations

import os

import torch

from nestor_b200.ops import reference as _ref
from nestor_b200.ops.reference import (  # noqa: F401  (plans + pure helpers are shared)
    ColumnPlan, DepthKeyCache, ExpertPlan, NS_COEFFS, RoutingTape, apply_rope, rope_tables, set_routing_tape,
)

_FORCE_REF = os.environ.get("NESTOR_B200_REFERENCE_OPS") == "1"
_cuda_mod = None


def cuda_ops():
    """The kernel namespace (imports and, if needed, builds the extension)."""

    global _cuda_mod
    if _cuda_mod is None:
        from nestor_b200.ops import cuda as _c
        _cuda_mod = _c
    return _cuda_mod


def launch_count() -> int:
    """Kernels of the in-tree library launched so far in this process."""

    from nestor_b200.ops import _lib
    return _lib.LAUNCHES


def oracle_path_report() -> dict[str, int]:
    """Calls that ran as PyTorch statements on CUDA tensors (op name -> count): a shape or option beyond a kernel's
    built-in limits (these warn the first time and raise under ``NESTOR_B200_STRICT=1``), or an op that has no fused
    kernel (the plain-residual and history-attention topologies). An empty dict means every op of the process ran
    on the sm_100a kernels.
    """

    return cuda_ops().oracle_path_report() if _cuda_mod is not None else {}


_oracle_depth = 0


class oracle_ops:
    """``with ops.oracle_ops():`` run the PyTorch statement of every op on any device.

    The kernels compute in bf16 with fp32 accumulation. Code that wants full-precision arithmetic on a GPU (fp32
    evaluation, numerics comparisons) asks for the oracle explicitly with this context; nothing selects it behind
    the caller's back.
    """

    def __enter__(self):
        global _oracle_depth
        _oracle_depth += 1
        return self

    def __exit__(self, *exc):
        global _oracle_depth
        _oracle_depth -= 1
        return False


def use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REF and _oracle_depth == 0


def _dispatch(name: str):
    ref_fn = getattr(_ref, name)

    def op(*args, **kwargs):
        first = next(a for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor)
                     or (isinstance(a, (list, tuple)) and len(a) > 0 and isinstance(a[0], torch.Tensor)))
        probe = first[0] if isinstance(first, (list, tuple)) else first
        if use_kernels(probe):
            fn = getattr(cuda_ops(), name, None)
            if fn is None:
                raise RuntimeError(f"ops.{name} has no sm_100a kernel body; CUDA tensors never take the PyTorch "
                                   "statement silently (set NESTOR_B200_REFERENCE_OPS=1 to run the oracle on a GPU)")
            return fn(*args, **kwargs)
        return ref_fn(*args, **kwargs)

    op.__name__ = name
    op.__doc__ = ref_fn.__doc__
    return op


def _eager(name: str, report_as: str):
    """An op without a fused kernel: the PyTorch statement on any device, counted in ``oracle_path_report()`` when
    it runs on CUDA tensors beside the kernels (the options that use it are outside the registered cells)."""

    ref_fn = getattr(_ref, name)

    def op(*args, **kwargs):
        first = next(a for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor)
                     or (isinstance(a, (list, tuple)) and len(a) > 0 and isinstance(a[0], torch.Tensor)))
        probe = first[0] if isinstance(first, (list, tuple)) else first
        if use_kernels(probe):
            cuda_ops().note_eager(report_as)
        return ref_fn(*args, **kwargs)

    op.__name__ = name
    op.__doc__ = ref_fn.__doc__
    return op


# The two halves of ``depth_read_norm`` as separate equations: test oracles (the registered cells call the fused op).
rmsnorm = _ref.rmsnorm
depth_read = _ref.depth_read
# what the plain-residual and history-attention topologies call: no fused kernel, counted when run on a GPU
stream_rmsnorm = _eager("rmsnorm", "rmsnorm")
depth_attention = _eager("depth_attention", "depth_attention")
depth_read_norm = _dispatch("depth_read_norm")
grad_sink = _dispatch("grad_sink")
mid_source = _dispatch("mid_source")
layer_combine = _dispatch("layer_combine")
block_exit = _dispatch("block_exit")
router_scores = _dispatch("router_scores")
route_topk = _dispatch("route_topk")
route_selected = _dispatch("route_selected")
build_column_plan = _dispatch("build_column_plan")
build_expert_plan = _dispatch("build_expert_plan")
column_attention = _dispatch("column_attention")
dense_attention = _dispatch("dense_attention")
expert_bank = _dispatch("expert_bank")
dense_swiglu = _dispatch("dense_swiglu")
lm_head_ce = _dispatch("lm_head_ce")
newton_schulz = _dispatch("newton_schulz")
