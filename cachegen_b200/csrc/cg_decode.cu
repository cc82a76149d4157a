// Arithmetic decoder kernels: one thread per stream, 128 adjacent channels of one row per block.
//
// The per-stream loop lives in cg_coder.cuh; this file stages tables, offsets and scales around it
// and writes either raw symbols (the torchac_cuda entry points) or dequantised 16-bit KV (fused path).
#include "cg_common.cuh"

namespace cg {

// Rows of a staged table: entries 0 .. lp-2 are searched (the entry after the last symbol stands for
// 2^16 and is never read), padded up to the span of the search.
__host__ __device__ inline int table_rows(int lp, int levels) {
    return (1 << levels) > lp - 1 ? (1 << levels) : lp - 1;
}

// ---- symbol-output kernels (decode_fast_prefsum / decode_fast_new) -----------------------------------
struct SymDecodeParams {
    const int16_t *cdf;
    const uint8_t *bytes;
    int64_t nbytes;          // total bytes addressable from `bytes`
    const int64_t *prefsum;  // mode 0
    const int32_t *lengths;  // mode 1
    int64_t stream_stride;   // mode 1
    uint8_t *out;
    int64_t o0, o1, o2;
    int ntokens, nchannels, lp;
    int32_t *status;
};

template <int LEVELS, bool POW2, int MODE>
__global__ void __launch_bounds__(kGroup) decode_symbols_kernel(const SymDecodeParams p) {
    extern __shared__ uint32_t tab[];
    const int tid = threadIdx.x;
    const int row = blockIdx.y;
    const int c = blockIdx.x * kGroup + tid;
    // the lanes that decode together, taken while the warp is still converged
    const uint32_t lanes = __ballot_sync(0xFFFFFFFFu, c < p.nchannels);
    if (c >= p.nchannels) return;  // no block barrier in this kernel
    const int64_t g = static_cast<int64_t>(row) * p.nchannels + c;
    int64_t start, len;
    if (MODE == 0) {
        start = g ? p.prefsum[g - 1] : 0;
        len = p.prefsum[g] - start;
    } else {
        start = g * p.stream_stride;
        len = p.lengths[g];
        if (len > p.stream_stride) len = p.stream_stride;
    }
    bool bad = false;
    if (len < 0) { len = 0; bad = true; }
    if (start < 0) { start = 0; len = 0; bad = true; }
    if (start > p.nbytes) { start = p.nbytes; bad = true; }
    if (start + len > p.nbytes) { len = p.nbytes - start; bad = true; }
    if (len > (1 << 20)) len = 1 << 20;
    if (bad && p.status) atomicOr(p.status, CG_S_BAD_LENGTHS);

    const int rows = table_rows(p.lp, LEVELS);
    stage_table_column(tab, p.cdf + g * p.lp, p.lp, rows, tid);
    uint8_t *o = p.out + row * p.o0 + c * p.o2;
    const int64_t o1 = p.o1;
    const uint32_t col = smem_addr(tab + tid);
    auto emit = [&](uint32_t a) {
        *o = static_cast<uint8_t>((a - col) / kRowBytes);
        o += o1;
    };
    decode_stream<LEVELS, POW2>(Smem{}, col, p.lp - 2, p.bytes + start, static_cast<uint32_t>(len), p.ntokens,
                                lanes, emit);
}

// ---- one warp per stream (kept for comparison) -------------------------------------------------------------
// The layout usually drawn for a GPU arithmetic decoder: a warp owns one stream, lane m holds table
// entry m in a register, a ballot over "(span * cdf[m]) >> 16 <= value - low" finds the symbol and two
// shuffles fetch its scaled bounds.  It needs no shared memory and no search loop, but all 32 lanes
// repeat the stream's serial range update, so it spends about 30 warp instructions per symbol where
// the thread-per-stream kernels spend about 70 per 32 symbols.  Same results; tables of at most 33
// entries; prefix-sum stream layout only.
__global__ void __launch_bounds__(kGroup) decode_symbols_warp_kernel(const SymDecodeParams p, int nrows) {
    const int lane = threadIdx.x & 31;
    const int64_t g = (static_cast<int64_t>(blockIdx.x) * kGroup + threadIdx.x) >> 5;
    if (g >= static_cast<int64_t>(nrows) * p.nchannels) return;
    const int row = static_cast<int>(g / p.nchannels), c = static_cast<int>(g % p.nchannels);
    int64_t start = g ? p.prefsum[g - 1] : 0;
    int64_t len = p.prefsum[g] - start;
    bool bad = false;
    if (len < 0) { len = 0; bad = true; }
    if (start < 0) { start = 0; len = 0; bad = true; }
    if (start > p.nbytes) { start = p.nbytes; bad = true; }
    if (start + len > p.nbytes) { len = p.nbytes - start; bad = true; }
    if (len > (1 << 20)) len = 1 << 20;
    if (bad && lane == 0 && p.status) atomicOr(p.status, CG_S_BAD_LENGTHS);

    const int maxsym = p.lp - 2;
    const uint32_t c16 = lane <= maxsym
                             ? static_cast<uint32_t>(static_cast<uint16_t>(__ldg(p.cdf + g * p.lp + lane))) << 16
                             : 0u;
    BitWindow bw;
    DecoderState st;
    st.low = 0u;
    st.span32 = 0u;
    st.offset = bw.open(p.bytes + start, static_cast<uint32_t>(len));
    uint8_t *o = p.out + row * p.o0 + c * p.o2;
    for (int i = 0; i < p.ntokens; ++i) {
        const uint32_t f = scale_exact(st.span32, c16);
        const uint32_t votes = __ballot_sync(0xFFFFFFFFu, lane <= maxsym && f <= st.offset);
        const int sym = 31 - __clz(static_cast<int>(votes | 1u));  // entry 0 is always taken
        if (lane == 0) o[i * p.o1] = static_cast<uint8_t>(sym);
        if (i == p.ntokens - 1) break;
        const uint32_t flo = __shfl_sync(0xFFFFFFFFu, f, sym);
        const uint32_t fnext = __shfl_sync(0xFFFFFFFFu, f, (sym + 1) & 31);
        st.update(flo, sym == maxsym ? st.span32 : fnext, bw);
        if (bw.low_water()) bw.refill();
    }
}

// ---- fused decode + dequantise + KV-layout store --------------------------------------------------------
struct FusedDecodeParams {
    int njobs, nlayers, nheads, head_size, nchannels, lp, nslab;
    int delta_group;         // 0: every token is coded on its own (the reference's behaviour)
    const float *res_bins;   // anchor-token delta: residual bin count per row, <= 0 for rows without it
    const float *bins;
    int64_t o_layer, o_kv, o_token, o_head;
    int32_t *status;
    cg_decode_job jobs[CG_MAX_DECODE_JOBS];
};

template <int LEVELS, bool POW2, int SCALE_DT, int OUT_DT>
__global__ void __launch_bounds__(kGroup) decode_dequant_kernel(const __grid_constant__ FusedDecodeParams p) {
    extern __shared__ uint32_t smem[];
    __shared__ float scale_f[kSubTokens];
    __shared__ float lut[CG_MAX_LP];
    __shared__ int warp_sums[kGroup / 32];

    const cg_decode_job &job = p.jobs[blockIdx.z];
    const int tid = threadIdx.x;
    const int row = blockIdx.y;
    const int c = blockIdx.x * kGroup + tid;
    const bool active = c < p.nchannels;
    const uint32_t lanes = __ballot_sync(0xFFFFFFFFu, active);  // taken while the warp is still converged
    const int ntok = job.ntokens;
    const int layer = row % p.nlayers, kv = row / p.nlayers;
    const int64_t g = static_cast<int64_t>(row) * p.nchannels + c;

    // stream offsets: group base + exclusive scan of this block's lengths (cachegen_decoder.py:70)
    int len = 0;
    if (active)
        len = job.length_kind == CG_LENGTHS_U16 ? static_cast<int>(__ldg(static_cast<const uint16_t *>(job.lengths) + g))
                                                : __ldg(static_cast<const int32_t *>(job.lengths) + g);
    bool bad = false;
    if (len < 0) { len = 0; bad = true; }
    if (len > (1 << 20)) { len = 1 << 20; bad = true; }
    const int excl = block_exclusive_scan_128(len, warp_sums, tid, nullptr);
    int64_t start = __ldg(job.group_off + static_cast<int64_t>(row) * p.nslab + blockIdx.x) + excl;
    if (start < 0) { start = 0; len = 0; bad = true; }
    if (start > job.nbytes) { start = job.nbytes; bad = true; }
    if (start + len > job.nbytes) { len = static_cast<int>(job.nbytes - start); bad = true; }
    if (bad && active && p.status) atomicOr(p.status, CG_S_BAD_LENGTHS);

    // per-token scales of this row and the row's (s - Cq) / Cq table (cachegen_decoder.py:30-32)
    const uint16_t *sc = static_cast<const uint16_t *>(kv ? job.scales_v : job.scales_k) +
                         static_cast<int64_t>(layer) * job.scale_stride;
    for (int t = tid; t < ntok; t += kGroup) scale_f[t] = Half16<SCALE_DT>::to_float(__ldg(sc + t));
    if (tid < p.lp - 1) {
        const float cq = half_range(__ldg(p.bins + row));
        lut[tid] = __fdiv_rn(__fsub_rn(static_cast<float>(tid), cq), cq);
    }
    const int rows = table_rows(p.lp, LEVELS);
    if (job.table_kind == CG_TABLES_SPARSE) {  // the whole block: the counts are found by a scan of the masks
        const int nrows = 2 * p.nlayers;
        const int cq = static_cast<int>(half_range(__ldg(p.bins + row)));
        const uint8_t *base = static_cast<const uint8_t *>(job.tables);
        const int64_t off_masks = (static_cast<int64_t>(nrows) * p.nslab + 1) * 4 + 15 & ~int64_t{15};
        const int64_t off_counts = off_masks + (__ldg(job.table_row_off + nrows) + 15 & ~int64_t{15});
        uint32_t mask = 0;
        bool inside = true;
        if (active) {
            const int width = 2 * cq <= 16 ? 2 : 4;
            const int64_t at_mask = off_masks + __ldg(job.table_row_off + row) + static_cast<int64_t>(c) * width;
            inside = at_mask >= 0 && at_mask + width <= job.tables_nbytes;
            if (inside)
                mask = width == 2 ? __ldg(reinterpret_cast<const uint16_t *>(base + at_mask))
                                  : __ldg(reinterpret_cast<const uint32_t *>(base + at_mask));
            if (2 * cq < 32) mask &= (1u << (2 * cq)) - 1u;
        }
        __syncthreads();  // warp_sums is free again
        const int before = block_exclusive_scan_128(__popc(mask), warp_sums, tid, nullptr);
        const int64_t at = off_counts +
                           __ldg(reinterpret_cast<const uint32_t *>(base) + static_cast<int64_t>(row) * p.nslab + blockIdx.x) +
                           before;
        const bool fits = inside && off_counts <= job.tables_nbytes && at + __popc(mask) <= job.tables_nbytes;
        if (!fits && active && p.status) atomicOr(p.status, CG_S_BAD_TABLE);
        if (active)
            stage_table_column_from_sparse(smem, mask, fits ? base + at : nullptr, cq, job.scale_stride, p.lp,
                                           rows + 1, tid);
    } else if (active) {
        if (job.table_kind == CG_TABLES_COUNTS) {
            const int cq = static_cast<int>(half_range(__ldg(p.bins + row)));
            const int64_t at = __ldg(job.table_row_off + row) + c;
            const bool fits = cq >= 0 && at >= 0 && at + static_cast<int64_t>(2 * cq - 1) * p.nchannels < job.tables_nbytes;
            if (!fits && p.status) atomicOr(p.status, CG_S_BAD_TABLE);
            stage_table_column_from_counts(smem, static_cast<const uint8_t *>(job.tables) + (fits ? at : 0), p.nchannels,
                                           fits ? cq : 0, job.scale_stride, p.lp, rows + 1, tid);
        } else {
            stage_table_column(smem, static_cast<const int16_t *>(job.tables) + g * p.lp, p.lp, rows + 1, tid);
        }
    }
    __syncthreads();
    if (!active) return;

    const int h = c / p.head_size, d = c - h * p.head_size;
    uint16_t *o = static_cast<uint16_t *>(job.out) + layer * p.o_layer + kv * p.o_kv + h * p.o_head + d;
    int64_t o_token = p.o_token;
    const uint32_t col = smem_addr(smem + tid);
    // entry m of the row's (s - Cq)/Cq table is at lut + 4m = lut + (a - col)/128 = (a >> 7) + lut_k,
    // because a - col is a multiple of 512
    uint32_t lut_k = smem_addr(lut) - (col >> 7), sc_a = smem_addr(scale_f);
    int ntok_r = ntok;
    // keep the loop's invariants in registers instead of re-deriving them from kernel parameters
    asm volatile("" : "+l"(o_token), "+r"(lut_k), "+r"(sc_a), "+r"(ntok_r));
    auto emit = [&](uint32_t a) {
        // ((sym - Cq) / Cq) * max in fp32, then one round-to-nearest cast (cachegen_decoder.py:30-33,171-173)
        const float v = __fmul_rn(ldsf32((a >> 7) + lut_k), ldsf32(sc_a));
        *o = Half16<OUT_DT>::from_float(v);
        o += o_token;
        sc_a += 4u;
    };
    decode_stream<LEVELS, POW2>(Smem{}, col, p.lp - 2, job.bytes + start, static_cast<uint32_t>(len), ntok_r,
                                lanes, emit);
}

// ---- the same with NS adjacent channels per thread ----------------------------------------------------------
// A block still covers one 128-channel group of one row, with 128 / NS threads: thread t decodes
// channels NS*t .. NS*t + NS-1 side by side (NS independent dependency chains per thread; loop
// control, the warp vote and the token's scale are paid once per NS symbols) and writes their 16-bit
// values with one 2*NS-byte store.  Channel NS*t + i keeps its table in column t + i * (128 / NS), so a
// warp still reads 32 different banks whatever entries its lanes are at.  The search depth is chosen
// per block from the row's bin count (see decode_streams); the result does not depend on it.
// Needs a head size and output strides that are multiples of NS and output pointers aligned to 2*NS bytes.
template <int OUT_DT>
__device__ __forceinline__ uint32_t pack_pair(float v0, float v1);
template <>
__device__ __forceinline__ uint32_t pack_pair<CG_F16>(float v0, float v1) {
    const __half2 h = __floats2half2_rn(v0, v1);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<CG_BF16>(float v0, float v1) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Shared memory (the tables) allows 12 blocks per SM at the usual table length of 33; asking for no
// more leaves the compiler 80 registers a thread, which it needs to interleave the NS chains.
constexpr int kMultiBlocksPerSM = 12;

// DELTA (anchor-token delta, see cg_decode_dequant_delta): in rows with residual bins every token that is
// not the first of its group of delta_group adds its value, ((sym - Cq_a) / Cq_r) * max, to its
// anchor's value as the KV dtype holds it; the sum is cast to the output type.
template <int NS, int OUT_DT, bool DELTA>
__global__ void __launch_bounds__(kGroup / NS, kMultiBlocksPerSM)
decode_dequant_multi_kernel(const __grid_constant__ FusedDecodeParams p, int scale_dt, int full_levels) {
    constexpr int kThreads = kGroup / NS;
    constexpr int kWarps = kThreads / 32;
    extern __shared__ uint32_t smem[];
    __shared__ float scale_f[kSubTokens];
    __shared__ float lut[(DELTA ? 2 : 1) * CG_MAX_LP];  // DELTA: the residual tokens' table follows the anchors'
    __shared__ int warp_sums[kWarps];

    const cg_decode_job &job = p.jobs[blockIdx.z];
    const int tid = threadIdx.x;
    const int row = blockIdx.y;
    const int c0 = blockIdx.x * kGroup + NS * tid;  // nchannels is a multiple of NS: all NS channels exist or none
    const bool active = c0 < p.nchannels;
    const uint32_t lanes = __ballot_sync(0xFFFFFFFFu, active);
    const int ntok = job.ntokens;
    const int layer = row % p.nlayers, kv = row / p.nlayers;
    const int64_t g = static_cast<int64_t>(row) * p.nchannels + c0;

    // stream offsets: group base + exclusive scan of this block's lengths (cachegen_decoder.py:70)
    int len[NS];
    bool bad = false;
    int len_sum = 0;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        len[i] = 0;
        if (active)
            len[i] = job.length_kind == CG_LENGTHS_U16
                         ? static_cast<int>(__ldg(static_cast<const uint16_t *>(job.lengths) + g + i))
                         : __ldg(static_cast<const int32_t *>(job.lengths) + g + i);
        if (len[i] < 0) { len[i] = 0; bad = true; }
        if (len[i] > (1 << 20)) { len[i] = 1 << 20; bad = true; }
        len_sum += len[i];
    }
    const int excl = block_exclusive_scan<kWarps>(len_sum, warp_sums, tid, nullptr);
    int64_t start[NS];
    start[0] = __ldg(job.group_off + static_cast<int64_t>(row) * p.nslab + blockIdx.x) + excl;
#pragma unroll
    for (int i = 1; i < NS; ++i) start[i] = start[i - 1] + len[i - 1];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        if (start[i] < 0) { start[i] = 0; len[i] = 0; bad = true; }
        if (start[i] > job.nbytes) { start[i] = job.nbytes; bad = true; }
        if (start[i] + len[i] > job.nbytes) { len[i] = static_cast<int>(job.nbytes - start[i]); bad = true; }
    }
    if (bad && active && p.status) atomicOr(p.status, CG_S_BAD_LENGTHS);

    // per-token scales of this row and the row's (s - Cq) / Cq table (cachegen_decoder.py:30-32)
    const uint16_t *sc = static_cast<const uint16_t *>(kv ? job.scales_v : job.scales_k) +
                         static_cast<int64_t>(layer) * job.scale_stride;
    for (int t = tid; t < ntok; t += kThreads) scale_f[t] = half_bits_to_float(__ldg(sc + t), scale_dt);
    const float cqf = half_range(__ldg(p.bins + row));
    for (int m = tid; m < p.lp - 1; m += kThreads) lut[m] = __fdiv_rn(__fsub_rn(static_cast<float>(m), cqf), cqf);
    uint32_t group_mask = 0xFFFFFFFFu;  // token index & group_mask == 0: an anchor (every token without delta)
    if (DELTA) {
        float cqr = 0.0f;
        bool on = false;
        if (p.res_bins) {
            const float rb = __ldg(p.res_bins + row);
            cqr = half_range(rb);
            on = rb > 0.0f && cqr >= 1.0f && cqr <= cqf;
        }
        if (on) {
            group_mask = static_cast<uint32_t>(p.delta_group) * 4u - 1u;  // on four times the token index
            for (int m = tid; m < p.lp - 1; m += kThreads)
                lut[CG_MAX_LP + m] = __fdiv_rn(__fsub_rn(static_cast<float>(m), cqf), cqr);
        } else {
            group_mask = 0u;
        }
    }
    const int cq = cqf >= 0.0f && cqf < 64.0f ? static_cast<int>(cqf) : 64;
    const int rows = table_rows(p.lp, full_levels < 2 ? 2 : full_levels);  // the register levels read entries 1..3
    uint32_t *tabs[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) tabs[i] = smem + tid + i * kThreads;
    if (job.table_kind == CG_TABLES_SPARSE) {  // the whole block: the counts are found by a scan of the masks
        const int nrows = 2 * p.nlayers;
        const uint8_t *base = static_cast<const uint8_t *>(job.tables);
        const int64_t off_masks = (static_cast<int64_t>(nrows) * p.nslab + 1) * 4 + 15 & ~int64_t{15};
        const int64_t off_counts = off_masks + (__ldg(job.table_row_off + nrows) + 15 & ~int64_t{15});
        uint32_t mask[NS];
        int nset[NS], nset_sum = 0;
        bool inside = true;
        const int width = 2 * cq <= 16 ? 2 : 4;
        const int64_t at_mask = off_masks + __ldg(job.table_row_off + row) + static_cast<int64_t>(c0) * width;
        if (active) inside = at_mask >= 0 && at_mask + NS * width <= job.tables_nbytes;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            mask[i] = 0;
            if (active && inside)
                mask[i] = width == 2 ? __ldg(reinterpret_cast<const uint16_t *>(base + at_mask) + i)
                                     : __ldg(reinterpret_cast<const uint32_t *>(base + at_mask) + i);
            if (2 * cq < 32) mask[i] &= (1u << (2 * cq)) - 1u;
            nset[i] = __popc(mask[i]);
            nset_sum += nset[i];
        }
        __syncthreads();  // warp_sums is free again
        const int before = block_exclusive_scan<kWarps>(nset_sum, warp_sums, tid, nullptr);
        int64_t at = off_counts +
                     __ldg(reinterpret_cast<const uint32_t *>(base) + static_cast<int64_t>(row) * p.nslab + blockIdx.x) +
                     before;
        const bool fits = inside && off_counts <= job.tables_nbytes && at + nset_sum <= job.tables_nbytes;
        if (!fits && active && p.status) atomicOr(p.status, CG_S_BAD_TABLE);
        if (active) {
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                stage_table_column_from_sparse(tabs[i], mask[i], fits ? base + at : nullptr, cq, job.scale_stride, p.lp,
                                               rows + 1, 0);
                at += nset[i];
            }
        }
    } else if (active) {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            if (job.table_kind == CG_TABLES_COUNTS) {
                const int64_t at = __ldg(job.table_row_off + row) + c0 + i;
                const bool fits = at >= 0 && at + static_cast<int64_t>(2 * cq - 1) * p.nchannels < job.tables_nbytes;
                if (!fits && p.status) atomicOr(p.status, CG_S_BAD_TABLE);
                stage_table_column_from_counts(tabs[i], static_cast<const uint8_t *>(job.tables) + (fits ? at : 0),
                                               p.nchannels, fits ? cq : 0, job.scale_stride, p.lp, rows + 1, 0);
            } else {
                stage_table_column(tabs[i], static_cast<const int16_t *>(job.tables) + (g + i) * p.lp, p.lp, rows + 1, 0);
            }
        }
    }
    __syncthreads();
    if (!active) return;

    const int h = c0 / p.head_size, d = c0 - h * p.head_size;
    uint16_t *o = static_cast<uint16_t *>(job.out) + layer * p.o_layer + kv * p.o_kv + h * p.o_head + d;
    uint32_t col[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) col[i] = smem_addr(tabs[i]);
    // entry m of the row's (s - Cq)/Cq table is at lut + 4m = (a >> 7) + lut_k for an entry address a
    // of column 0, because a - col is a multiple of 512; column i starts 4 * kThreads bytes further,
    // which adds kThreads / 32 to (a >> 7)
    uint32_t lut_k = smem_addr(lut) - (col[0] >> 7);
    int64_t o_token = p.o_token;
    uint32_t sc_a = smem_addr(scale_f);
    int ntok_r = ntok;
    // keep the loop's invariants in registers instead of re-deriving them from kernel parameters
    asm volatile("" : "+l"(o_token), "+r"(lut_k), "+r"(sc_a), "+r"(ntok_r));
    float anchor[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) anchor[i] = 0.0f;
    auto emit = [&](const uint32_t (&a)[NS], uint32_t t4) {
        // ((sym - Cq) / Cq) * max in fp32, then one round-to-nearest cast (cachegen_decoder.py:30-33,171-173)
        const float s = ldsf32(sc_a);
        float v[NS];
        if (!DELTA || (t4 & group_mask) == 0u) {
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                v[i] = __fmul_rn(ldsf32((a[i] >> 7) + lut_k - i * (kThreads / 32)), s);
                if (DELTA)  // what the encoder subtracted from the group's other tokens: the value in the KV dtype
                    anchor[i] = scale_dt == CG_BF16 ? Half16<CG_BF16>::to_float(Half16<CG_BF16>::from_float(v[i]))
                                                    : Half16<CG_F16>::to_float(Half16<CG_F16>::from_float(v[i]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < NS; ++i)
                v[i] = __fadd_rn(anchor[i], __fmul_rn(ldsf32((a[i] >> 7) + lut_k - i * (kThreads / 32) + 4u * CG_MAX_LP), s));
        }
        if (NS == 2) {
            *reinterpret_cast<uint32_t *>(o) = pack_pair<OUT_DT>(v[0], v[1]);
        } else {
            *reinterpret_cast<uint2 *>(o) = make_uint2(pack_pair<OUT_DT>(v[0], v[1]), pack_pair<OUT_DT>(v[2 % NS], v[3 % NS]));
        }
        o += o_token;
        sc_a += 4u;
    };
    const int maxsym = p.lp - 2;
    const int fl = fast_levels_for(2 * cq + 1, full_levels);
    const int top = (1 << fl) - 1;
    const uint32_t det = smem_addr(smem) + static_cast<uint32_t>(top < maxsym ? top : maxsym) * kRowBytes;
    const uint8_t *streams[NS];
    uint32_t lens[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        streams[i] = job.bytes + start[i];
        lens[i] = static_cast<uint32_t>(len[i]);
    }
    switch (fl) {
    case 2: decode_streams<2, NS>(Smem{}, col, det, maxsym, full_levels, streams, lens, ntok_r, lanes, emit); break;
    case 3: decode_streams<3, NS>(Smem{}, col, det, maxsym, full_levels, streams, lens, ntok_r, lanes, emit); break;
    case 4: decode_streams<4, NS>(Smem{}, col, det, maxsym, full_levels, streams, lens, ntok_r, lanes, emit); break;
    case 5: decode_streams<5, NS>(Smem{}, col, det, maxsym, full_levels, streams, lens, ntok_r, lanes, emit); break;
    default: decode_streams<6, NS>(Smem{}, col, det, maxsym, full_levels, streams, lens, ntok_r, lanes, emit); break;
    }
}

// ---- launch helpers -------------------------------------------------------------------------------------
// dynamic shared memory of a decoder block: the streams' table columns
static size_t table_bytes(int lp, int levels) {
    return static_cast<size_t>(table_rows(lp, levels) + 1) * kRowBytes;  // +1: the row read past the last symbol
}

// Instantiated search depths: exact power-of-two tables for lp = 9, 17, 33 and clamped searches of
// depth 3..6 for every other lp <= 64.
template <int MODE>
static int launch_symbols(const SymDecodeParams &p, int nrows, cudaStream_t st) {
    const int need = search_levels(p.lp);
    const bool pow2 = (1 << need) == p.lp - 1;
    const dim3 grid((p.nchannels + kGroup - 1) / kGroup, nrows), block(kGroup);
#define CG_LAUNCH_SYM(L, P2)                                                                              \
    do {                                                                                                  \
        const size_t smem = table_bytes(p.lp, L);                                                         \
        if (smem > 48 * 1024)                                                                             \
            cudaFuncSetAttribute(decode_symbols_kernel<L, P2, MODE>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));    \
        decode_symbols_kernel<L, P2, MODE><<<grid, block, smem, st>>>(p);                                 \
    } while (0)
    if (pow2 && need == 5) CG_LAUNCH_SYM(5, true);
    else if (pow2 && need == 4) CG_LAUNCH_SYM(4, true);
    else if (pow2 && need == 3) CG_LAUNCH_SYM(3, true);
    else if (need <= 3) CG_LAUNCH_SYM(3, false);
    else if (need == 4) CG_LAUNCH_SYM(4, false);
    else if (need == 5) CG_LAUNCH_SYM(5, false);
    else CG_LAUNCH_SYM(6, false);
#undef CG_LAUNCH_SYM
    return check_launch();
}

template <int SCALE_DT, int OUT_DT>
static int launch_fused(const FusedDecodeParams &p, cudaStream_t st) {
    const int need = search_levels(p.lp);
    const bool pow2 = (1 << need) == p.lp - 1;
    const dim3 grid(p.nslab, 2 * p.nlayers, p.njobs), block(kGroup);
#define CG_LAUNCH_FUSED(L, P2)                                                                            \
    do {                                                                                                  \
        const size_t smem = table_bytes(p.lp, L);                                                         \
        if (smem > 48 * 1024)                                                                             \
            cudaFuncSetAttribute(decode_dequant_kernel<L, P2, SCALE_DT, OUT_DT>,                          \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));    \
        decode_dequant_kernel<L, P2, SCALE_DT, OUT_DT><<<grid, block, smem, st>>>(p);                     \
    } while (0)
    if (pow2 && need == 5) CG_LAUNCH_FUSED(5, true);
    else if (pow2 && need == 4) CG_LAUNCH_FUSED(4, true);
    else if (pow2 && need == 3) CG_LAUNCH_FUSED(3, true);
    else if (need <= 3) CG_LAUNCH_FUSED(3, false);
    else if (need == 4) CG_LAUNCH_FUSED(4, false);
    else if (need == 5) CG_LAUNCH_FUSED(5, false);
    else CG_LAUNCH_FUSED(6, false);
#undef CG_LAUNCH_FUSED
    return check_launch();
}

// The NS-channels-per-thread kernel needs the NS channels of a thread in one head and aligned packed stores.
static bool multi_layout_ok(const FusedDecodeParams &p, int ns) {
    if ((p.head_size | p.o_layer | p.o_kv | p.o_token | p.o_head) & (ns - 1)) return false;
    for (int j = 0; j < p.njobs; ++j)
        if (reinterpret_cast<uintptr_t>(p.jobs[j].out) & (2 * ns - 1)) return false;
    return true;
}

template <int NS, int OUT_DT, bool DELTA>
static int launch_fused_multi(const FusedDecodeParams &p, int scale_dt, cudaStream_t st) {
    const int full = search_levels(p.lp);
    const size_t smem = table_bytes(p.lp, full < 2 ? 2 : full);
    const dim3 grid(p.nslab, 2 * p.nlayers, p.njobs), block(kGroup / NS);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(decode_dequant_multi_kernel<NS, OUT_DT, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    decode_dequant_multi_kernel<NS, OUT_DT, DELTA><<<grid, block, smem, st>>>(p, scale_dt, full);
    return check_launch();
}

}  // namespace cg

using namespace cg;

static int check_coder_shape(int nrows, int ntokens, int nchannels, int lp) {
    if (nrows <= 0 || ntokens <= 0 || nchannels <= 0) return CG_E_SHAPE;
    if (ntokens > CG_MAX_TOKENS_PER_STREAM) return CG_E_TOKENS;
    if (lp < 2 || lp > CG_MAX_LP) return CG_E_LP;
    if (nrows > 65535) return CG_E_SHAPE;
    return CG_OK;
}

extern "C" int cg_decode_prefsum(const int16_t *cdf, const uint8_t *bytes, int64_t nbytes,
                                 const int64_t *prefsum, uint8_t *out, const int64_t out_strides[3],
                                 int nrows, int ntokens, int nchannels, int lp, int32_t *status,
                                 void *stream) {
    if (!cdf || !prefsum || !out || !out_strides || (!bytes && nbytes > 0)) return CG_E_NULL;
    if (nbytes < 0) return CG_E_SHAPE;
    if (int rc = check_coder_shape(nrows, ntokens, nchannels, lp)) return rc;
    SymDecodeParams p{cdf, bytes, nbytes, prefsum, nullptr, 0, out, out_strides[0], out_strides[1],
                      out_strides[2], ntokens, nchannels, lp, status};
    return launch_symbols<0>(p, nrows, static_cast<cudaStream_t>(stream));
}

extern "C" int cg_decode_prefsum_warp(const int16_t *cdf, const uint8_t *bytes, int64_t nbytes,
                                      const int64_t *prefsum, uint8_t *out, const int64_t out_strides[3],
                                      int nrows, int ntokens, int nchannels, int lp, int32_t *status,
                                      void *stream) {
    if (!cdf || !prefsum || !out || !out_strides || (!bytes && nbytes > 0)) return CG_E_NULL;
    if (nbytes < 0) return CG_E_SHAPE;
    if (int rc = check_coder_shape(nrows, ntokens, nchannels, lp)) return rc;
    if (lp > 33) return CG_E_LP;
    SymDecodeParams p{cdf, bytes, nbytes, prefsum, nullptr, 0, out, out_strides[0], out_strides[1],
                      out_strides[2], ntokens, nchannels, lp, status};
    const int64_t nstreams = static_cast<int64_t>(nrows) * nchannels;
    const int64_t blocks = (nstreams * 32 + kGroup - 1) / kGroup;
    if (blocks > 0x7FFFFFFF) return CG_E_SHAPE;
    decode_symbols_warp_kernel<<<static_cast<unsigned>(blocks), kGroup, 0, static_cast<cudaStream_t>(stream)>>>(p, nrows);
    return check_launch();
}

extern "C" int cg_decode_padded(const int16_t *cdf, const uint8_t *streams, int64_t stream_stride,
                                const int32_t *lengths, uint8_t *out, const int64_t out_strides[3],
                                int nrows, int ntokens, int nchannels, int lp, int32_t *status,
                                void *stream) {
    if (!cdf || !streams || !lengths || !out || !out_strides) return CG_E_NULL;
    if (stream_stride <= 0) return CG_E_SHAPE;
    if (int rc = check_coder_shape(nrows, ntokens, nchannels, lp)) return rc;
    SymDecodeParams p{cdf, streams, static_cast<int64_t>(nrows) * nchannels * stream_stride, nullptr,
                      lengths, stream_stride, out, out_strides[0], out_strides[1], out_strides[2],
                      ntokens, nchannels, lp, status};
    return launch_symbols<1>(p, nrows, static_cast<cudaStream_t>(stream));
}

// Checks the arguments of the fused decode and fills the kernel parameters; launches nothing.
static int fused_params(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads, int head_size, int lp,
                        const float *bins, int scale_dtype, int out_dtype, int64_t o_layer, int64_t o_kv,
                        int64_t o_token, int64_t o_head, int32_t *status, FusedDecodeParams &p) {
    if (!jobs_host || !bins) return CG_E_NULL;
    if (njobs <= 0 || nlayers <= 0 || nheads <= 0 || head_size <= 0) return CG_E_SHAPE;
    if (njobs > CG_MAX_DECODE_JOBS) return CG_E_CAPACITY;
    if (lp < 2 || lp > CG_MAX_LP) return CG_E_LP;
    if (nlayers > 32767) return CG_E_SHAPE;  // 2 * nlayers rows are a grid dimension
    if (static_cast<int64_t>(nheads) * head_size > 0x7FFFFFFF - kGroup) return CG_E_SHAPE;
    if ((scale_dtype != CG_F16 && scale_dtype != CG_BF16) || (out_dtype != CG_F16 && out_dtype != CG_BF16))
        return CG_E_DTYPE;
    p.njobs = njobs;
    p.nlayers = nlayers;
    p.nheads = nheads;
    p.head_size = head_size;
    p.nchannels = nheads * head_size;
    p.lp = lp;
    p.nslab = (p.nchannels + kGroup - 1) / kGroup;
    p.delta_group = 0;
    p.res_bins = nullptr;
    p.bins = bins;
    p.o_layer = o_layer;
    p.o_kv = o_kv;
    p.o_token = o_token;
    p.o_head = o_head;
    p.status = status;
    for (int j = 0; j < njobs; ++j) {
        const cg_decode_job &jb = jobs_host[j];
        if (!jb.tables || !jb.lengths || !jb.group_off || !jb.scales_k || !jb.scales_v || !jb.out ||
            (!jb.bytes && jb.nbytes > 0) || (jb.table_kind != CG_TABLES_CDF && !jb.table_row_off))
            return CG_E_NULL;
        if ((jb.table_kind != CG_TABLES_CDF && jb.table_kind != CG_TABLES_COUNTS && jb.table_kind != CG_TABLES_SPARSE) ||
            (jb.length_kind != CG_LENGTHS_I32 && jb.length_kind != CG_LENGTHS_U16))
            return CG_E_SHAPE;
        if (jb.table_kind == CG_TABLES_SPARSE) {
            if (jb.tables_nbytes < (static_cast<int64_t>(2 * nlayers) * p.nslab + 1) * 4) return CG_E_CAPACITY;
            if (reinterpret_cast<uintptr_t>(jb.tables) & 3) return CG_E_ALIGN;
        }
        if (jb.table_kind == CG_TABLES_COUNTS && jb.tables_nbytes <= 0) return CG_E_CAPACITY;
        if (jb.ntokens <= 0 || jb.nbytes < 0) return CG_E_SHAPE;
        if (jb.ntokens > CG_MAX_TOKENS_PER_STREAM) return CG_E_TOKENS;
        p.jobs[j] = jb;
    }
    return CG_OK;
}

static int launch_fused_any(const FusedDecodeParams &p, int scale_dtype, int out_dtype, cudaStream_t st) {
    if (p.delta_group > 0) {  // only the two-channels-per-thread kernel knows about anchors
        if (!multi_layout_ok(p, 2)) return CG_E_ALIGN;
        return out_dtype == CG_F16 ? launch_fused_multi<2, CG_F16, true>(p, scale_dtype, st)
                                   : launch_fused_multi<2, CG_BF16, true>(p, scale_dtype, st);
    }
    if (multi_layout_ok(p, 2))
        return out_dtype == CG_F16 ? launch_fused_multi<2, CG_F16, false>(p, scale_dtype, st)
                                   : launch_fused_multi<2, CG_BF16, false>(p, scale_dtype, st);
    if (scale_dtype == CG_F16 && out_dtype == CG_F16) return launch_fused<CG_F16, CG_F16>(p, st);
    if (scale_dtype == CG_F16 && out_dtype == CG_BF16) return launch_fused<CG_F16, CG_BF16>(p, st);
    if (scale_dtype == CG_BF16 && out_dtype == CG_F16) return launch_fused<CG_BF16, CG_F16>(p, st);
    return launch_fused<CG_BF16, CG_BF16>(p, st);
}

extern "C" int cg_decode_dequant(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                                 int head_size, int lp, const float *bins, int scale_dtype,
                                 int out_dtype, int64_t o_layer, int64_t o_kv, int64_t o_token,
                                 int64_t o_head, int32_t *status, void *stream) {
    FusedDecodeParams p;
    if (int rc = fused_params(jobs_host, njobs, nlayers, nheads, head_size, lp, bins, scale_dtype, out_dtype,
                              o_layer, o_kv, o_token, o_head, status, p))
        return rc;
    return launch_fused_any(p, scale_dtype, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int cg_decode_dequant_delta(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                                       int head_size, int lp, const float *bins, int delta_group,
                                       const float *res_bins, int scale_dtype, int out_dtype, int64_t o_layer,
                                       int64_t o_kv, int64_t o_token, int64_t o_head, int32_t *status, void *stream) {
    FusedDecodeParams p;
    if (int rc = fused_params(jobs_host, njobs, nlayers, nheads, head_size, lp, bins, scale_dtype, out_dtype,
                              o_layer, o_kv, o_token, o_head, status, p))
        return rc;
    if (delta_group) {
        if (!res_bins) return CG_E_NULL;
        if (delta_group < 2 || delta_group > CG_MAX_TOKENS_PER_STREAM || CG_MAX_TOKENS_PER_STREAM % delta_group)
            return CG_E_SHAPE;
        p.delta_group = delta_group;
        p.res_bins = res_bins;
    }
    return launch_fused_any(p, scale_dtype, out_dtype, static_cast<cudaStream_t>(stream));
}

// ---- decode without a caller-provided workspace --------------------------------------------------------------
// Group offsets for callers that cannot allocate (see the header): a fixed array in the library's
// own device image.  In host code `g_static_group_off` is only a handle for the runtime, not a
// device address; the address each device gave the array is looked up once per device below.
static __device__ __align__(256) int64_t g_static_group_off[CG_STATIC_OFFSET_ENTRIES];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
int64_t *g_static_ptr[kMaxDevices];  // device address of g_static_group_off, per device

// Address of the array on the current device; set up on the first call per device.
int static_group_off(int64_t **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_cuda_error(e);
    if (dev < 0 || dev >= kMaxDevices) return CG_E_CAPACITY;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_group_off);
        if (e != cudaSuccess) return set_cuda_error(e);
        g_static_ptr[dev] = static_cast<int64_t *>(p);
    }
    *out = g_static_ptr[dev];
    return CG_OK;
}
}  // namespace

extern "C" int cg_decode_dequant_static(const cg_decode_job *jobs_host, int njobs, int nlayers, int nheads,
                                        int head_size, int lp, const float *bins, int scale_dtype,
                                        int out_dtype, int64_t o_layer, int64_t o_kv, int64_t o_token,
                                        int64_t o_head, int32_t *status, void *stream) {
    if (!jobs_host || !bins) return CG_E_NULL;
    if (njobs <= 0 || nlayers <= 0 || nheads <= 0 || head_size <= 0) return CG_E_SHAPE;
    if (njobs > CG_MAX_DECODE_JOBS) return CG_E_CAPACITY;
    if (nlayers > 32767 || static_cast<int64_t>(nheads) * head_size > 0x7FFFFFFF - kGroup) return CG_E_SHAPE;
    const int nchannels = nheads * head_size;
    const int64_t ngroups = static_cast<int64_t>(2 * nlayers) * ((nchannels + kGroup - 1) / kGroup);
    if (ngroups * njobs > CG_STATIC_OFFSET_ENTRIES) return CG_E_CAPACITY;
    int64_t *scratch = nullptr;
    if (int rc = static_group_off(&scratch)) return rc;
    cg_decode_job jobs[CG_MAX_DECODE_JOBS];
    for (int j = 0; j < njobs; ++j) {
        jobs[j] = jobs_host[j];
        jobs[j].group_off = scratch + j * ngroups;
    }
    // every argument check of the fused decode comes before the first launch into the shared array
    FusedDecodeParams p;
    if (int rc = fused_params(jobs, njobs, nlayers, nheads, head_size, lp, bins, scale_dtype, out_dtype, o_layer,
                              o_kv, o_token, o_head, status, p))
        return rc;
    if (int rc = cg_decode_offsets(jobs, njobs, 2 * nlayers, nchannels, scratch, status, stream)) return rc;
    return launch_fused_any(p, scale_dtype, out_dtype, static_cast<cudaStream_t>(stream));
}
