// Sparse form of the byte-count tables (CG_TABLES_SPARSE in cachegen_b200.h): for every (row, channel)
// a bit mask of the non-centre symbols that occur in the chunk, and the non-zero counts alone.
// Most channels of a key row use three or four symbols out of 15 or 31, so the table set shrinks to
// about 40 % of the byte counts; it travels with the streams, so that is what a decode from host
// memory saves on the bus.  No counterpart in the reference, whose tables are int16 [2L, C, Lp].
#include "cg_common.cuh"

namespace cg {

// bits of one channel: bit j set when stored symbol j (centre skipped) has a non-zero count
__device__ __forceinline__ uint32_t count_mask(const uint8_t *cnt, int64_t stride, int nstored) {
    uint32_t m = 0;
    for (int j = 0; j < nstored; ++j) m |= (__ldg(cnt + j * stride) ? 1u : 0u) << j;
    return m;
}

__device__ __forceinline__ int stored_symbols(const float *bins, int row) {
    const int n = 2 * static_cast<int>(half_range(__ldg(bins + row)));
    return n < 32 ? n : 32;  // wider rows cannot be written in this form: the caller rules them out
}

// pass 1: masks out, and the number of non-zero counts of every (row, group)
__global__ void __launch_bounds__(kGroup) sparse_masks_kernel(const uint8_t *counts, const int64_t *count_row_off,
                                                              const float *bins, int nchannels, uint8_t *masks,
                                                              const int64_t *mask_row_off, uint32_t *group_bytes) {
    __shared__ int warp_sums[kGroup / 32];
    const int tid = threadIdx.x, row = blockIdx.y, c = blockIdx.x * kGroup + tid;
    const int nstored = stored_symbols(bins, row);
    uint32_t m = 0;
    if (c < nchannels) {
        m = count_mask(counts + __ldg(count_row_off + row) + c, nchannels, nstored);
        uint8_t *mrow = masks + __ldg(mask_row_off + row);
        if (nstored <= 16) reinterpret_cast<uint16_t *>(mrow)[c] = static_cast<uint16_t>(m);
        else reinterpret_cast<uint32_t *>(mrow)[c] = m;
    }
    int total = 0;
    block_exclusive_scan_128(__popc(m), warp_sums, tid, &total);
    if (tid == 0) group_bytes[static_cast<int64_t>(row) * gridDim.x + blockIdx.x] = static_cast<uint32_t>(total);
}

// pass 2: exclusive scan of the n group sizes in place, total into entry n (one block)
__global__ void __launch_bounds__(1024) sparse_scan_kernel(uint32_t *group_off, int n) {
    __shared__ uint32_t part[1024];
    const int tid = threadIdx.x;
    const int per = (n + 1023) / 1024;
    const int lo = tid * per, hi = min(n, lo + per);
    uint32_t s = 0;
    for (int i = lo; i < hi; ++i) s += group_off[i];
    part[tid] = s;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
        const uint32_t v = tid >= d ? part[tid - d] : 0u;
        __syncthreads();
        part[tid] += v;
        __syncthreads();
    }
    uint32_t run = part[tid] - s;
    for (int i = lo; i < hi; ++i) {
        const uint32_t v = group_off[i];
        group_off[i] = run;
        run += v;
    }
    if (tid == 1023) group_off[n] = part[1023];
}

// pass 3: the non-zero counts of every channel to their place
__global__ void __launch_bounds__(kGroup) sparse_pack_kernel(const uint8_t *counts, const int64_t *count_row_off,
                                                             const float *bins, int nchannels,
                                                             const uint32_t *group_off, uint8_t *out) {
    __shared__ int warp_sums[kGroup / 32];
    const int tid = threadIdx.x, row = blockIdx.y, c = blockIdx.x * kGroup + tid;
    const int nstored = stored_symbols(bins, row);
    const uint8_t *cnt = counts + __ldg(count_row_off + row) + c;
    const uint32_t m = c < nchannels ? count_mask(cnt, nchannels, nstored) : 0u;
    const int excl = block_exclusive_scan_128(__popc(m), warp_sums, tid, nullptr);
    uint8_t *o = out + group_off[static_cast<int64_t>(row) * gridDim.x + blockIdx.x] + excl;
    for (int j = 0; j < nstored; ++j)
        if ((m >> j) & 1u) *o++ = __ldg(cnt + static_cast<int64_t>(j) * nchannels);
}

}  // namespace cg

using namespace cg;

extern "C" int cg_pack_sparse_tables(const uint8_t *counts, const int64_t *count_row_off, const float *bins,
                                     int nrows, int nchannels, uint32_t *group_off_out, void *masks_out,
                                     const int64_t *mask_row_off, uint8_t *counts_out, void *stream) {
    if (!counts || !count_row_off || !bins || !group_off_out || !masks_out || !mask_row_off || !counts_out)
        return CG_E_NULL;
    if (nrows <= 0 || nchannels <= 0 || nrows > 65535) return CG_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(masks_out) & 3) || (reinterpret_cast<uintptr_t>(group_off_out) & 3))
        return CG_E_ALIGN;
    const int nslab = (nchannels + kGroup - 1) / kGroup;
    if (static_cast<int64_t>(nrows) * nslab >= (int64_t{1} << 30)) return CG_E_SHAPE;  // offsets are uint32 counts
    const dim3 grid(nslab, nrows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    sparse_masks_kernel<<<grid, kGroup, 0, st>>>(counts, count_row_off, bins, nchannels,
                                                 static_cast<uint8_t *>(masks_out), mask_row_off, group_off_out);
    if (int rc = check_launch()) return rc;
    sparse_scan_kernel<<<1, 1024, 0, st>>>(group_off_out, nrows * nslab);
    if (int rc = check_launch()) return rc;
    sparse_pack_kernel<<<grid, kGroup, 0, st>>>(counts, count_row_off, bins, nchannels, group_off_out, counts_out);
    return check_launch();
}
