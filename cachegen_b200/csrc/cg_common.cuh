// Shared device helpers of the sm_100a CacheGen codec kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/cachegen_b200.h"
#include "cg_coder.cuh"

namespace cg {

constexpr int kGroup = kGroupChannels;           // streams (threads) per coder block
constexpr int kRowBytes = kTableRowBytes;        // bytes of one table row in shared memory
static_assert(kGroup == CG_GROUP_CHANNELS, "header and kernels disagree on the group size");
constexpr int kSubTokens = CG_MAX_TOKENS_PER_STREAM;

// ---- error plumbing -------------------------------------------------------------------------
int set_cuda_error(cudaError_t e);  // records the text, returns CG_E_CUDA
inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? CG_OK : set_cuda_error(e);
}

// ---- search depth for a table of lp entries ---------------------------------------------------
// Symbols are 0 .. lp-2.  levels = smallest n with 2^n >= lp-1; pow2 when 2^n == lp-1.
inline int search_levels(int lp) {
    int n = 0;
    while ((1 << n) < lp - 1) n++;
    return n;
}

// ---- small PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ float ldsf32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- table staging ----------------------------------------------------------------------------
// Every thread owns one (row, channel) table.  It is kept in shared memory as tab[m][tid] =
// cdf[m] << 16 so that lane i always hits bank i, whatever entry m each lane is at.  Each thread
// fills (and later reads) only its own column, so no block barrier is needed.  Only the entries of
// the symbols, 0 .. lp-2, are staged; the rows above them hold kTablePadding, which a search step
// of the decoder takes for "above the target" (see decode_streams in cg_coder.cuh).
constexpr uint32_t kTablePadding = 0xFFFFFFFFu;
__device__ __forceinline__ void stage_table_column(uint32_t *tab, const int16_t *cdf_row, int lp,
                                                   int rows, int tid) {
    const int n = lp - 1 < rows ? lp - 1 : rows;
    for (int m = 0; m < n; ++m)
        tab[m * kGroup + tid] = static_cast<uint32_t>(static_cast<uint16_t>(__ldg(cdf_row + m))) << 16;
    for (int m = n; m < rows; ++m) tab[m * kGroup + tid] = kTablePadding;
}

// The same column from the byte counts of the non-centre symbols (CG_TABLES_COUNTS):
// cdf[i] = (uint16)((0xFFFF - max_bins) * #{sym < i} / ntokens) + i, as calculate_cdf builds it
// (cal_cdf.cu:11-15,40-49 in the reference).  cnt points at this channel's first count; counts of one
// symbol are `stride` bytes apart; cq = bins // 2 - 1 is the centre symbol, whose count is implied.
__device__ __forceinline__ void stage_table_column_from_counts(uint32_t *tab, const uint8_t *cnt, int64_t stride,
                                                               int cq, int ntokens, int lp, int rows, int tid) {
    const int max_bins = lp - 1;
    uint32_t others = 0;
    for (int j = 0; j < 2 * cq; ++j) others += __ldg(cnt + j * stride);
    const uint32_t centre = static_cast<uint32_t>(ntokens) - others;
    const uint32_t scale = 0xFFFFu - static_cast<uint32_t>(max_bins);
    const uint32_t total = static_cast<uint32_t>(ntokens) & 0xFFFFu;
    const bool pow2 = (total & (total - 1u)) == 0u;
    const int sh = 31 - __clz(static_cast<int>(total | 1u));
    const int n = lp - 1 < rows ? lp - 1 : rows;
    uint32_t cum = 0;
    for (int i = 0; i < n; ++i) {
        const uint32_t prod = scale * (cum & 0xFFFFu);
        const uint32_t nv = total ? (pow2 ? (prod >> sh) : (prod / total)) : 0u;
        tab[i * kGroup + tid] = ((nv + static_cast<uint32_t>(i)) & 0xFFFFu) << 16;
        uint32_t count = 0;
        if (i < cq) count = __ldg(cnt + i * stride);
        else if (i == cq) count = centre;
        else if (i <= 2 * cq) count = __ldg(cnt + (i - 1) * stride);
        cum += count;
    }
    for (int i = n; i < rows; ++i) tab[i * kGroup + tid] = kTablePadding;
}

// The same column from the sparse byte counts (CG_TABLES_SPARSE): `mask` has bit j set when stored
// symbol j (centre skipped) has a non-zero count, and `nz` points at those counts in rising symbol
// order (nullptr: read them all as zero).
__device__ __forceinline__ void stage_table_column_from_sparse(uint32_t *tab, uint32_t mask, const uint8_t *nz, int cq,
                                                               int ntokens, int lp, int rows, int tid) {
    const int max_bins = lp - 1;
    if (2 * cq < 32) mask &= (1u << (2 * cq)) - 1u;
    if (!nz) mask = 0u;
    uint32_t others = 0;
    for (int k = __popc(mask) - 1; k >= 0; --k) others += __ldg(nz + k);
    const uint32_t centre = static_cast<uint32_t>(ntokens) - others;
    const uint32_t scale = 0xFFFFu - static_cast<uint32_t>(max_bins);
    const uint32_t total = static_cast<uint32_t>(ntokens) & 0xFFFFu;
    const bool pow2 = (total & (total - 1u)) == 0u;
    const int sh = 31 - __clz(static_cast<int>(total | 1u));
    const int n = lp - 1 < rows ? lp - 1 : rows;
    uint32_t cum = 0;
    for (int i = 0; i < n; ++i) {
        const uint32_t prod = scale * (cum & 0xFFFFu);
        const uint32_t nv = total ? (pow2 ? (prod >> sh) : (prod / total)) : 0u;
        tab[i * kGroup + tid] = ((nv + static_cast<uint32_t>(i)) & 0xFFFFu) << 16;
        uint32_t count = 0;
        if (i == cq) {
            count = centre;
        } else if (i <= 2 * cq) {
            if (mask & 1u) count = __ldg(nz++);
            mask >>= 1;
        }
        cum += count;
    }
    for (int i = n; i < rows; ++i) tab[i * kGroup + tid] = kTablePadding;
}

// ---- block-wide exclusive scan over 32 * NWARPS ints --------------------------------------------
// warp_sums: shared int[NWARPS].  Returns the exclusive prefix of `v` across the block.
template <int NWARPS>
__device__ __forceinline__ int block_exclusive_scan(int v, int *warp_sums, int tid, int *total) {
    const int lane = tid & 31, w = tid >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += n;
    }
    if (lane == 31) warp_sums[w] = incl;
    __syncthreads();
    int base = 0, all = 0;
#pragma unroll
    for (int i = 0; i < NWARPS; ++i) {
        const int s = warp_sums[i];
        if (i < w) base += s;
        all += s;
    }
    if (total) *total = all;
    return base + incl - v;
}
__device__ __forceinline__ int block_exclusive_scan_128(int v, int *warp_sums, int tid, int *total) {
    return block_exclusive_scan<kGroup / 32>(v, warp_sums, tid, total);
}

template <int DT> struct Half16;
template <> struct Half16<CG_F16> {
    static __device__ __forceinline__ float to_float(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    static __device__ __forceinline__ uint16_t from_float(float f) { return __half_as_ushort(__float2half_rn(f)); }
};
template <> struct Half16<CG_BF16> {
    static __device__ __forceinline__ float to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
    static __device__ __forceinline__ uint16_t from_float(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
};

__device__ __forceinline__ float half_bits_to_float(uint16_t b, int dtype) {
    return dtype == CG_BF16 ? Half16<CG_BF16>::to_float(b) : Half16<CG_F16>::to_float(b);
}

// Cq of do_dequantize / MAX of torch_quant_vectorized: bins // 2 - 1 on a float tensor.
__device__ __forceinline__ float half_range(float bins) { return __fsub_rn(floorf(__fdiv_rn(bins, 2.0f)), 1.0f); }

}  // namespace cg
