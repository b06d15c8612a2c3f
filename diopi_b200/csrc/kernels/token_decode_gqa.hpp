// The single-pass grouped-query decode kernel (token_decode_gqa.cu) as seen by the decode dispatch in token_decode.cu.
#pragma once

#include "kernels.hpp"

namespace b200 {
namespace k {

// Scratch the kernel needs for these arguments; 0 when they do not qualify (not fused mode, kv_group outside 2..128,
// a dtype other than fp16/bf16, a head_dim other than 64 or 128, rows that are not dense and 16-byte aligned).
int64_t decode_gqa_workspace_bytes(const DecodeArgs& a, int sm_count, int max_smem);
// Launches the kernel and the merge kernel after it; false (nothing launched) when the arguments do not qualify.
bool launch_decode_gqa(const DecodeArgs& a, void* ws, int sm_count, int max_smem, cudaStream_t st);

}  // namespace k
}  // namespace b200
