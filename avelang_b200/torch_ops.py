"""The ``torch.ops.avelang_gdn`` operator namespace: the PyTorch-extension face of libave_gdn_b200.so.

Each operator is declared here with its schema and implemented (CUDA dispatch key) by the function that fills the
C argument block and calls the library's ``extern "C"`` entry point on torch's current stream; the public functions
in ``gdn.py`` / ``gemm.py`` validate, allocate and then call these operators, so the operators are the one path to the
kernels.  Operators write into tensors the caller passes (``out``, state pools) and return nothing, like the C entry
points they wrap; mutated arguments carry an alias annotation in the schema."""
from __future__ import annotations

import torch

NAMESPACE = "avelang_gdn"
_library = torch.library.Library(NAMESPACE, "DEF")

SCHEMAS = {
    "chunk_prefill": "(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor(a!) out, float scale, "
                     "Tensor? initial_state, Tensor(b!)? final_state, Tensor? cu_seqlens, Tensor? state_indices, "
                     "Tensor? z, Tensor? norm_weight, float norm_eps, bool qk_l2norm, int max_seqlen, Tensor? out_peers) -> ()",
    "decode_step": "(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor(a!) out, float scale, "
                   "Tensor? initial_state, Tensor(b!)? final_state, Tensor? cu_seqlens, Tensor? state_indices, "
                   "Tensor? z, Tensor? norm_weight, float norm_eps, bool qk_l2norm) -> ()",
    "gated_rmsnorm": "(Tensor x, Tensor z, Tensor? weight, float eps, bool gate_first, Tensor(a!) out) -> ()",
    "conv1d_silu": "(Tensor x, Tensor weight, Tensor? bias, Tensor? cu_seqlens, Tensor(a!) out) -> ()",
    "conv1d_update": "(Tensor x, Tensor(a!) conv_state, Tensor weight, Tensor? bias, Tensor? state_indices, Tensor(b!) out) -> ()",
    "gate_beta": "(Tensor a, Tensor b, Tensor A_log, Tensor dt_bias, Tensor(a!) g, Tensor(b!) beta) -> ()",
    "gemm_bf16_nt": "(Tensor A, Tensor B, Tensor(a!) out) -> ()",
    "gemm_scatter": "(Tensor A, Tensor B, Tensor(a!) stage, Tensor stage_peers, int rank, int rows_per_owner) -> ()",
    "gemm_reduce_push": "(Tensor stage, Tensor out_peers, Tensor(a!) out, int rank, int M, int rows_per_owner) -> ()",
    "recurrent_backward": "(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor d_o, float scale, Tensor? initial_state, "
                          "Tensor? d_final_state, Tensor? cu_seqlens, Tensor(a!) dq, Tensor(b!) dk, Tensor(c!) dv, Tensor(d!) dg, "
                          "Tensor(e!) dbeta, Tensor(f!)? d_initial_state) -> ()",
    "decode_layer_step": "(Tensor proj, Tensor conv_w, Tensor? conv_bias, Tensor(a!) conv_state, Tensor A_log, Tensor dt_bias, "
                         "Tensor? norm_weight, Tensor(b!) state_pool, Tensor? state_indices, Tensor(c!) out, int Hk, int Hv, "
                         "float scale, float norm_eps, bool gate_first) -> ()",
}
for _name, _schema in SCHEMAS.items():
    _library.define(_name + _schema)


def implement(name: str):
    """Decorator: registers the CUDA implementation of ``torch.ops.avelang_gdn.<name>``."""
    def deco(fn):
        _library.impl(name, fn, "CUDA")
        return fn
    return deco


def op(name: str):
    return getattr(getattr(torch.ops, NAMESPACE), name)
