// extern "C" boundary of libave_gdn_b200.so: argument validation and dispatch.  No device allocation,
// no synchronisation, nothing thrown across the boundary.
#include "common.cuh"

namespace ave {
thread_local int g_last_cuda_error = 0;

int launch_decode(const AveGdnArgs& a, cudaStream_t stream);
int launch_prefill_simt(const AveGdnArgs& a, cudaStream_t stream);
size_t prefill_simt_workspace_bytes(const AveGdnArgs& a);
int launch_prefill_tc(const AveGdnArgs& a, cudaStream_t stream, bool plain);
size_t prefill_tc_workspace_bytes(const AveGdnArgs& a, bool plain);
int prefill_tc_launch_count(const AveGdnArgs& a, bool plain);
int launch_gated_rmsnorm(const AveGdnNormArgs& a, cudaStream_t stream);
int launch_conv1d_silu(const AveConvArgs& a, cudaStream_t stream);
int launch_gate_beta(const AveGateArgs& a, cudaStream_t stream);
int launch_conv1d_update(const AveConvUpdateArgs& a, cudaStream_t stream);
int launch_gemm_bf16_nt(const AveGemmArgs& a, cudaStream_t stream);
int launch_gemm_bf16_nt_scatter(const AveGemmReduceArgs& a, cudaStream_t stream);
int launch_gemm_reduce_push(const AveGemmReduceArgs& a, cudaStream_t stream);
int launch_decode_layer(const AveGdnDecodeLayerArgs& a, cudaStream_t stream);
int launch_backward(const AveGdnBwdArgs& a, cudaStream_t stream);
size_t backward_workspace_bytes(const AveGdnBwdArgs& a);

static size_t prefill_ws_bytes(const AveGdnArgs& a) {
  return a.dk == 128 ? prefill_tc_workspace_bytes(a, false) : prefill_simt_workspace_bytes(a);
}

static int check_rows(const void* p, int64_t st, int64_t sh, int64_t sb, int elem_bytes) {
  if (!aligned16(p)) return AVE_GDN_MISALIGNED;
  if ((st * elem_bytes) % 16 || (sh * elem_bytes) % 16 || (sb * elem_bytes) % 16) return AVE_GDN_MISALIGNED;
  return AVE_GDN_OK;
}

static int validate_gdn(const AveGdnArgs* a, bool prefill) {
  if (a == nullptr || a->struct_size != sizeof(AveGdnArgs)) return AVE_GDN_INVALID_ARGUMENT;
  if (a->B < 0 || a->T < 0 || a->n_seqs < 0 || a->Hk <= 0 || a->Hv <= 0 || a->num_slots < 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->Hv % a->Hk != 0) return AVE_GDN_INVALID_ARGUMENT;
  if (!((a->dk == 128 && a->dv == 128) || (a->dk == 64 && a->dv == 64))) return AVE_GDN_UNSUPPORTED;
  if (a->cu_seqlens != nullptr && a->B != 1) return AVE_GDN_INVALID_ARGUMENT;
  if (a->cu_seqlens == nullptr && a->n_seqs != a->B) return AVE_GDN_INVALID_ARGUMENT;
  if (a->state_indices == nullptr && (a->initial_state || a->final_state) && a->num_slots < a->n_seqs) return AVE_GDN_INVALID_ARGUMENT;
  if ((int64_t)a->B * a->T == 0 || a->n_seqs == 0) return AVE_GDN_OK;
  if (!a->q || !a->k || !a->v || !a->g || !a->beta || !a->o) return AVE_GDN_INVALID_ARGUMENT;
  if (prefill && a->chunk != 64) return AVE_GDN_UNSUPPORTED;
  int rc;
  if ((rc = check_rows(a->q, a->q_stride_t, a->q_stride_h, a->q_stride_b, 2))) return rc;
  if ((rc = check_rows(a->k, a->k_stride_t, a->k_stride_h, a->k_stride_b, 2))) return rc;
  if ((rc = check_rows(a->v, a->v_stride_t, a->v_stride_h, a->v_stride_b, 2))) return rc;
  if ((rc = check_rows(a->o, a->o_stride_t, a->o_stride_h, a->o_stride_b, 2))) return rc;
  if (a->z && (rc = check_rows(a->z, a->z_stride_t, a->z_stride_h, a->z_stride_b, 2))) return rc;
  if (a->initial_state && !aligned16(a->initial_state)) return AVE_GDN_MISALIGNED;
  if (a->final_state && !aligned16(a->final_state)) return AVE_GDN_MISALIGNED;
  if ((reinterpret_cast<uintptr_t>(a->g) & 3u) || (reinterpret_cast<uintptr_t>(a->beta) & 3u)) return AVE_GDN_MISALIGNED;
  if (a->n_peers < 0 || (a->n_peers > 0 && a->o_peers == nullptr)) return AVE_GDN_INVALID_ARGUMENT;
  if (a->n_peers > 0 && (!prefill || a->z == nullptr || a->dk != 128)) return AVE_GDN_UNSUPPORTED;
  return AVE_GDN_OK;
}

// Argument checks of the prefill entry points, for translation units that define further prefill variants.
int validate_prefill_args(const AveGdnArgs* a) { return validate_gdn(a, true); }
}  // namespace ave

using namespace ave;

extern "C" {

int ave_gdn_abi_version(void) { return AVE_GDN_ABI_VERSION; }

int ave_gdn_last_cuda_error(void) { return g_last_cuda_error; }

const char* ave_gdn_status_string(int status) {
  switch (status) {
    case AVE_GDN_OK: return "ok";
    case AVE_GDN_INVALID_ARGUMENT: return "invalid argument";
    case AVE_GDN_UNSUPPORTED: return "unsupported shape";
    case AVE_GDN_MISALIGNED: return "pointer or stride not 16-byte aligned";
    case AVE_GDN_CUDA_ERROR: return "CUDA error";
    case AVE_GDN_WORKSPACE_TOO_SMALL: return "workspace too small";
    default: return "unknown status";
  }
}

size_t ave_gdn_prefill_workspace_bytes(const AveGdnArgs* args) {
  if (validate_gdn(args, true) != AVE_GDN_OK) return 0;
  return prefill_ws_bytes(*args);
}

int ave_gdn_prefill_launch_count(const AveGdnArgs* args) {
  if (validate_gdn(args, true) != AVE_GDN_OK) return 0;
  if ((int64_t)args->B * args->T == 0 || args->n_seqs == 0) return 0;
  if (args->dk == 128) return prefill_tc_launch_count(*args, false);
  return (args->cu_seqlens ? 1 : 0) + 2 + (args->z ? 1 : 0);  // chunk table, two passes, gated norm
}

int ave_gdn_chunk_prefill(const AveGdnArgs* args, void* stream) {
  const int rc = validate_gdn(args, true);
  if (rc != AVE_GDN_OK) return rc;
  if ((int64_t)args->B * args->T == 0 || args->n_seqs == 0) return AVE_GDN_OK;
  if (args->workspace == nullptr || !aligned16(args->workspace)) return AVE_GDN_INVALID_ARGUMENT;
  if (args->workspace_bytes < prefill_ws_bytes(*args)) return AVE_GDN_WORKSPACE_TOO_SMALL;
  // d = 128 runs on the tensor cores; d = 64 (the small CPU-reference shape) on the fp32 CUDA-core kernels
  if (args->dk == 128) return launch_prefill_tc(*args, reinterpret_cast<cudaStream_t>(stream), false);
  return launch_prefill_simt(*args, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_decode_step(const AveGdnArgs* args, void* stream) {
  const int rc = validate_gdn(args, false);
  if (rc != AVE_GDN_OK) return rc;
  if ((int64_t)args->B * args->T == 0 || args->n_seqs == 0) return AVE_GDN_OK;
  return launch_decode(*args, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_gated_rmsnorm(const AveGdnNormArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveGdnNormArgs) || a->rows < 0 || a->heads <= 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->d != 64 && a->d != 128) return AVE_GDN_UNSUPPORTED;
  if (a->rows == 0) return AVE_GDN_OK;
  if (!a->x || !a->z || !a->y) return AVE_GDN_INVALID_ARGUMENT;
  const int64_t strides[] = {a->x_stride_t, a->x_stride_h, a->z_stride_t, a->z_stride_h, a->y_stride_t, a->y_stride_h};
  const int64_t need = a->d == 128 ? 16 : 8;  // bytes a lane loads at once
  for (int64_t s : strides)
    if ((s * 2) % need) return AVE_GDN_MISALIGNED;
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->z) | reinterpret_cast<uintptr_t>(a->y)) & (uintptr_t)(need - 1)) return AVE_GDN_MISALIGNED;
  return launch_gated_rmsnorm(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_conv1d_silu(const AveConvArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveConvArgs) || a->B < 0 || a->T < 0 || a->C < 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->width < 2 || a->width > 4 || a->C % 8) return AVE_GDN_UNSUPPORTED;
  if (a->cu_seqlens != nullptr && (a->B != 1 || a->n_seqs <= 0)) return AVE_GDN_INVALID_ARGUMENT;
  if ((int64_t)a->B * a->T * a->C == 0) return AVE_GDN_OK;
  if (!a->x || !a->w || !a->y) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->x) || !aligned16(a->y) || (a->x_stride_t % 8) || (a->y_stride_t % 8) || (a->x_stride_b % 8) || (a->y_stride_b % 8))
    return AVE_GDN_MISALIGNED;
  return launch_conv1d_silu(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_conv1d_update(const AveConvUpdateArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveConvUpdateArgs) || a->n_seqs < 0 || a->C < 0 || a->num_slots < 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->width < 2 || a->width > 4 || a->C % 8) return AVE_GDN_UNSUPPORTED;
  if (a->n_seqs == 0 || a->C == 0) return AVE_GDN_OK;
  if (!a->x || !a->w || !a->y || !a->conv_state) return AVE_GDN_INVALID_ARGUMENT;
  if (a->state_indices == nullptr && a->num_slots < a->n_seqs) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->x) || !aligned16(a->y) || !aligned16(a->conv_state) || (a->x_stride % 8) || (a->y_stride % 8)) return AVE_GDN_MISALIGNED;
  return launch_conv1d_update(*a, reinterpret_cast<cudaStream_t>(stream));
}

static int validate_bwd(const AveGdnBwdArgs* a) {
  if (a == nullptr || a->struct_size != sizeof(AveGdnBwdArgs)) return AVE_GDN_INVALID_ARGUMENT;
  if (a->B < 0 || a->T < 0 || a->n_seqs < 0 || a->Hk <= 0 || a->Hv <= 0 || a->Hv % a->Hk != 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->dk != 128 || a->dv != 128) return AVE_GDN_UNSUPPORTED;
  if (a->cu_seqlens != nullptr && a->B != 1) return AVE_GDN_INVALID_ARGUMENT;
  if (a->cu_seqlens == nullptr && a->n_seqs != a->B) return AVE_GDN_INVALID_ARGUMENT;
  if ((int64_t)a->B * a->T == 0 || a->n_seqs == 0) return AVE_GDN_OK;
  if (!a->q || !a->k || !a->v || !a->g || !a->beta || !a->d_o || !a->d_q || !a->d_k || !a->d_v || !a->d_g || !a->d_beta) return AVE_GDN_INVALID_ARGUMENT;
  int rc;
  if ((rc = check_rows(a->q, a->q_stride_t, a->q_stride_h, a->q_stride_b, 2))) return rc;
  if ((rc = check_rows(a->k, a->k_stride_t, a->k_stride_h, a->k_stride_b, 2))) return rc;
  if ((rc = check_rows(a->v, a->v_stride_t, a->v_stride_h, a->v_stride_b, 2))) return rc;
  if ((rc = check_rows(a->d_o, a->do_stride_t, a->do_stride_h, a->do_stride_b, 2))) return rc;
  if (!aligned16(a->d_q) || !aligned16(a->d_k) || !aligned16(a->d_v)) return AVE_GDN_MISALIGNED;
  if ((a->initial_state && !aligned16(a->initial_state)) || (a->d_final_state && !aligned16(a->d_final_state)) ||
      (a->d_initial_state && !aligned16(a->d_initial_state)))
    return AVE_GDN_MISALIGNED;
  return AVE_GDN_OK;
}

size_t ave_gdn_backward_workspace_bytes(const AveGdnBwdArgs* a) {
  if (validate_bwd(a) != AVE_GDN_OK) return 0;
  return backward_workspace_bytes(*a);
}

int ave_gdn_recurrent_backward(const AveGdnBwdArgs* a, void* stream) {
  const int rc = validate_bwd(a);
  if (rc != AVE_GDN_OK) return rc;
  if ((int64_t)a->B * a->T == 0 || a->n_seqs == 0) return AVE_GDN_OK;
  if (a->workspace == nullptr || !aligned16(a->workspace)) return AVE_GDN_INVALID_ARGUMENT;
  if (a->workspace_bytes < backward_workspace_bytes(*a)) return AVE_GDN_WORKSPACE_TOO_SMALL;
  return launch_backward(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_decode_layer_step(const AveGdnDecodeLayerArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveGdnDecodeLayerArgs)) return AVE_GDN_INVALID_ARGUMENT;
  if (a->n_seqs < 0 || a->Hk <= 0 || a->Hv <= 0 || a->num_slots < 0 || a->Hv % a->Hk != 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->dk != 128 || a->dv != 128 || a->width < 2 || a->width > 4) return AVE_GDN_UNSUPPORTED;
  if (a->n_seqs == 0) return AVE_GDN_OK;
  if (!a->proj || !a->conv_w || !a->conv_state || !a->A_log || !a->dt_bias || !a->state_pool || !a->o) return AVE_GDN_INVALID_ARGUMENT;
  if (a->state_indices == nullptr && a->num_slots < a->n_seqs) return AVE_GDN_INVALID_ARGUMENT;
  const int64_t cols = 2 * (int64_t)a->Hk * a->dk + 2 * (int64_t)a->Hv * a->dv + 2 * a->Hv;
  if (a->proj_stride < cols || a->o_stride < (int64_t)a->Hv * a->dv) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->proj) || !aligned16(a->o) || !aligned16(a->state_pool) || !aligned16(a->conv_state) || (a->proj_stride % 8) ||
      (a->o_stride % 8))
    return AVE_GDN_MISALIGNED;
  return launch_decode_layer(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gdn_gate_beta(const AveGateArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveGateArgs) || a->rows < 0 || a->Hv <= 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->rows == 0) return AVE_GDN_OK;
  if (!a->a || !a->b || !a->A_log || !a->dt_bias || !a->g || !a->beta) return AVE_GDN_INVALID_ARGUMENT;
  return launch_gate_beta(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gemm_bf16_nt(const AveGemmArgs* a, void* stream) {
  if (a == nullptr || a->struct_size != sizeof(AveGemmArgs) || a->M < 0 || a->N < 0 || a->K < 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->M == 0 || a->N == 0) return AVE_GDN_OK;
  if (!a->a || !a->b || !a->c) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->c) || (a->lda % 8) || (a->ldb % 8) || (a->ldc % 8)) return AVE_GDN_MISALIGNED;
  if (a->K % 8 || a->K == 0) return AVE_GDN_UNSUPPORTED;
  return launch_gemm_bf16_nt(*a, reinterpret_cast<cudaStream_t>(stream));
}

static int validate_gemm_reduce(const AveGemmReduceArgs* a) {
  if (a == nullptr || a->struct_size != sizeof(AveGemmReduceArgs) || a->M < 0 || a->N < 0 || a->K < 0) return AVE_GDN_INVALID_ARGUMENT;
  if (a->n_ranks < 1 || a->n_ranks > 64 || a->rank < 0 || a->rank >= a->n_ranks) return AVE_GDN_INVALID_ARGUMENT;
  if (a->rows_per_owner <= 0 || a->rows_per_owner * a->n_ranks < a->M) return AVE_GDN_INVALID_ARGUMENT;
  if (!a->stage_peers || !a->stage || !a->out_peers) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->stage) || (a->N % 8) || (a->ldc % 8) || a->ldc < a->N) return AVE_GDN_MISALIGNED;
  return AVE_GDN_OK;
}

int ave_gemm_bf16_nt_scatter(const AveGemmReduceArgs* a, void* stream) {
  const int rc = validate_gemm_reduce(a);
  if (rc != AVE_GDN_OK) return rc;
  if (a->M == 0 || a->N == 0) return AVE_GDN_OK;
  if (!a->a || !a->b) return AVE_GDN_INVALID_ARGUMENT;
  if (!aligned16(a->a) || !aligned16(a->b) || (a->lda % 8) || (a->ldb % 8)) return AVE_GDN_MISALIGNED;
  if (a->K % 8 || a->K == 0) return AVE_GDN_UNSUPPORTED;
  return launch_gemm_bf16_nt_scatter(*a, reinterpret_cast<cudaStream_t>(stream));
}

int ave_gemm_reduce_push(const AveGemmReduceArgs* a, void* stream) {
  const int rc = validate_gemm_reduce(a);
  if (rc != AVE_GDN_OK) return rc;
  if (a->M == 0 || a->N == 0) return AVE_GDN_OK;
  return launch_gemm_reduce_push(*a, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
