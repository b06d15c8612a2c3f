// DestIndexCopyKV: out[dest_loc[t], :, :] = k[t, :, :].
// Replaces the single ATen index_put_ of impl/torch/functions/functions_lightllm.cpp:18-26.
// HBM-bound byte copy: 2*T*H*D*e bytes + T index loads. Rows are H*D*e bytes
// (8 KB at 32 heads x 128 x fp16), so the fast path moves 16-byte vectors with
// fully coalesced loads and stores; a strided element path covers everything else.
#include "dev_util.cuh"

namespace b200 {
namespace k {

namespace {

// One thread per 16-byte vector of a source row. Rows must be dense and 16-byte aligned.
__global__ void __launch_bounds__(256) copy_rows_vec16(CopyKVArgs a, int64_t vec_per_row, int64_t total_vec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec; i += stride) {
        const int64_t t = i / vec_per_row;
        const int64_t c = i - t * vec_per_row;
        int64_t slot = load_index(a.dest, t);
        if (slot < 0) slot += a.slots;  // index_put_ accepts negative indices
        if (slot < 0 || slot >= a.slots) {
            if (c == 0) report_status(a.status, 1);
            continue;
        }
        const uint4* s = reinterpret_cast<const uint4*>(static_cast<const char*>(a.src) + t * a.src_s0 * a.elem_bytes) + c;
        uint4* d = reinterpret_cast<uint4*>(static_cast<char*>(a.dst) + slot * a.dst_s0 * a.elem_bytes) + c;
        *d = __ldg(s);
    }
}

// One thread per element, any strides.
template <typename U>
__global__ void __launch_bounds__(256) copy_rows_elem(CopyKVArgs a, int64_t total) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t hd = a.H * a.D;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t t = i / hd;
        const int64_t r = i - t * hd;
        const int64_t h = r / a.D;
        const int64_t d = r - h * a.D;
        int64_t slot = load_index(a.dest, t);
        if (slot < 0) slot += a.slots;
        if (slot < 0 || slot >= a.slots) {
            if (r == 0) report_status(a.status, 1);
            continue;
        }
        const U* s = static_cast<const U*>(a.src) + t * a.src_s0 + h * a.src_s1 + d * a.src_s2;
        U* o = static_cast<U*>(a.dst) + slot * a.dst_s0 + h * a.dst_s1 + d * a.dst_s2;
        *o = *s;
    }
}

}  // namespace

void launch_dest_index_copy(const CopyKVArgs& a, cudaStream_t st) {
    const int64_t total = a.T * a.H * a.D;
    if (total == 0) return;
    const int64_t row_bytes = a.H * a.D * a.elem_bytes;
    const bool dense_rows = (a.D == 1 || (a.src_s2 == 1 && a.dst_s2 == 1)) && (a.H == 1 || (a.src_s1 == a.D && a.dst_s1 == a.D));
    const bool vec_ok = dense_rows && row_bytes % 16 == 0 && (a.src_s0 * a.elem_bytes) % 16 == 0 && (a.dst_s0 * a.elem_bytes) % 16 == 0 &&
                        (reinterpret_cast<uintptr_t>(a.src) % 16 == 0) && (reinterpret_cast<uintptr_t>(a.dst) % 16 == 0);
    if (vec_ok) {
        const int64_t vpr = row_bytes / 16;
        const int64_t tv = vpr * a.T;
        const int blocks = static_cast<int>(std::min<int64_t>((tv + 255) / 256, 148 * 16));
        copy_rows_vec16<<<blocks, 256, 0, st>>>(a, vpr, tv);
        return;
    }
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
    switch (a.elem_bytes) {
        case 2: copy_rows_elem<uint16_t><<<blocks, 256, 0, st>>>(a, total); break;
        case 4: copy_rows_elem<uint32_t><<<blocks, 256, 0, st>>>(a, total); break;
        case 8: copy_rows_elem<uint64_t><<<blocks, 256, 0, st>>>(a, total); break;
        default: copy_rows_elem<uint8_t><<<blocks, 256, 0, st>>>(a, total); break;
    }
}

}  // namespace k
}  // namespace b200
