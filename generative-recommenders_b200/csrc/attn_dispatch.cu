// Chooses between the tensor-core and the CUDA-core attention kernels and sizes their scratch.
#include "attn_plan.cuh"

namespace b200hstu {

bool attn_tc_layout_ok(const b200_hstu_attn_args &a, bool bwd, const char **why);
int64_t attn_tc_fwd_workspace_bytes(const b200_hstu_attn_args &a);
int64_t attn_tc_bwd_workspace_bytes(const b200_hstu_attn_args &a);

bool attn_tc_applicable(const b200_hstu_attn_args &a, bool bwd, const char **why) {
  if (a.dropout_ratio > 0.f && a.dropout_seed != nullptr) {
    *why = "dropout on the attention weights is only handled by the CUDA-core kernels";
    return false;
  }
  if (bwd && a.attn_scale != nullptr && a.attn_scale_numel > 1) {
    *why = "per-token attn_scale is only handled by the CUDA-core backward";
    return false;
  }
  return attn_tc_layout_ok(a, bwd, why);
}

// which: 0 = forward, 1 = backward, 2 = forward that also plans the backward
int64_t attn_tc_workspace_bytes(const b200_hstu_attn_args &a, int which) {
  // the forward's and the backward's scratch share the bias table
  if (which == 2)
    return attn_tc_fwd_workspace_bytes(a) + attn_tc_bwd_workspace_bytes(a) -
           bias_table_bytes(a.bias_by_distance, a.max_seq_len);
  return which == 1 ? attn_tc_bwd_workspace_bytes(a) : attn_tc_fwd_workspace_bytes(a);
}

}  // namespace b200hstu
