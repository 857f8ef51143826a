"""Kernel libraries under the reference project's namespace.

The reference ships its kernel libraries as modules of the ``avelang_kernels`` package and its callers import them as
``from avelang_kernels import <module>`` (benchmark/gemm/bench_amdgpu_gemm.py:4,
test/examples/gemm/amdgpu/test_amdgpu_gemm.py:7).  The same spelling reaches the B200 path:

    from avelang_kernels import gdn    # chunk_gated_delta_rule, fused_recurrent_gated_delta_rule, gated_rmsnorm, ...
    from avelang_kernels import gemm   # gemm_pipeline_transposed_b (counterpart of amdgpu_gemm.gemm_pipeline_transposed_b)

``avelang_kernels.gdn`` and ``avelang_kernels.gemm`` are the modules ``avelang_b200.gdn`` and ``avelang_b200.gemm``
themselves (one implementation under two import paths); importing them registers the ``torch.ops.avelang_gdn``
operators through which every entry point reaches the C library."""
import sys

from avelang_b200 import gdn, gemm

sys.modules[__name__ + ".gdn"] = gdn
sys.modules[__name__ + ".gemm"] = gemm

__all__ = ["gdn", "gemm"]
