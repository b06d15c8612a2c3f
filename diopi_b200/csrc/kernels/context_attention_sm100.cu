// Tensor-core causal prefill for sm_100a (tcgen05 + TMEM + TMA). Placeholder until the kernel
// lands: reports "not taken" so that every shape runs on the blockwise SIMT kernel.
#include "dev_util.cuh"

namespace b200 {
namespace k {

void launch_prefill_tc(const PrefillArgs& /*a*/, int /*sm_count*/, int /*max_smem*/, cudaStream_t /*st*/, bool* taken) { *taken = false; }

}  // namespace k
}  // namespace b200
