// Quantisation, histogram and CDF-table kernels.
//
//  * row_absmax_kernel      : per (row, token) amax(|x|) over all channels, the scale of
//                             torch_quant_vectorized (cachegen_encoder.py:55 in the reference);
//  * quantize_cdf_kernel    : per (row, 128-channel slab): quantise every token of the chunk with
//                             128-bit loads, write int8 symbols, count them with shared-memory
//                             atomics, and turn the counts into the reference's int16 tables
//                             (cachegen_encoder.py:54-57, cal_cdf.cu:29-49);
//  * symbol_cdf_kernel      : the stand-alone calculate_cdf on int8 symbols (cal_cdf.cu:17-59).
#include "cg_common.cuh"

namespace cg {

struct KvLayout {
    int64_t s_layer, s_kv, s_token, s_head;
    int nlayers, ntokens, nheads, head_size;
};

// |x| as an ordered integer: 16-bit float magnitudes compare like their bit patterns
__device__ __forceinline__ uint32_t absmax2(uint32_t best, uint32_t packed) {
    return __vmaxu2(best, packed & 0x7FFF7FFFu);
}

// One warp per (row, token).  scales[row, token] gets the 16-bit pattern of max|x|.
// Rows row0 .. row0 + nrows - 1.
template <int VEC>
__global__ void __launch_bounds__(256) row_absmax_kernel(const uint16_t *__restrict__ kv, const KvLayout L,
                                                         uint16_t *__restrict__ scales, int row0, int nrows) {
    int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<int64_t>(nrows) * L.ntokens) return;
    wid += static_cast<int64_t>(row0) * L.ntokens;
    const int row = static_cast<int>(wid / L.ntokens), t = static_cast<int>(wid % L.ntokens);
    const int layer = row % L.nlayers, j = row / L.nlayers;
    const uint16_t *base = kv + layer * L.s_layer + j * L.s_kv + t * L.s_token;
    uint32_t best = 0;
    if (VEC == 8) {
        const int per_head = L.head_size / 8;
        const int nvec = L.nheads * per_head;
        for (int v = lane; v < nvec; v += 32) {
            const int h = v / per_head, d = (v - h * per_head) * 8;
            const uint4 q = __ldg(reinterpret_cast<const uint4 *>(base + h * L.s_head + d));
            best = absmax2(absmax2(absmax2(absmax2(best, q.x), q.y), q.z), q.w);
        }
    } else {
        const int C = L.nheads * L.head_size;
        for (int c = lane; c < C; c += 32) {
            const int h = c / L.head_size, d = c - h * L.head_size;
            best = absmax2(best, __ldg(base + h * L.s_head + d));
        }
    }
    best = max(best & 0xFFFFu, best >> 16);
#pragma unroll
    for (int d = 16; d; d >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, d));
    if (lane == 0) scales[wid] = static_cast<uint16_t>(best);
}

// ---- anchor-token delta (no counterpart in the reference, see cg_quantize_cdf_delta in the header) -------
// What a decoder holds for one element of an anchor token: quantise as the plain path does, then
// ((sym - Cq) / Cq) * max in fp32 and one cast to the KV dtype.  lut[s] = (s - Cq) / Cq.
template <int DT>
__device__ __forceinline__ float anchor_value(uint16_t xa, float factor_a, float cqa, uint32_t keep, float max_a,
                                              const float *lut) {
    const float p = __fmul_rn(Half16<DT>::to_float(xa), factor_a);
    const uint32_t s = __float_as_uint(__fadd_rn(__fadd_rn(p, cqa), 8388608.0f)) & keep;
    return Half16<DT>::to_float(Half16<DT>::from_float(__fmul_rn(lut[s & 63u], max_a)));
}
// The residual of one element against its anchor, rounded to the KV dtype.
template <int DT>
__device__ __forceinline__ uint16_t residual_bits(uint16_t x, float anchor) {
    return Half16<DT>::from_float(__fsub_rn(Half16<DT>::to_float(x), anchor));
}
// A row is delta-coded when its residual bin count gives 1 <= Cq_r <= Cq_a.
__device__ __forceinline__ bool delta_row(const float *res_bins, int row, float cqa, float *cqr) {
    if (!res_bins) return false;
    const float rb = __ldg(res_bins + row);
    if (!(rb > 0.0f)) return false;
    *cqr = half_range(rb);
    return *cqr >= 1.0f && *cqr <= cqa;
}

// One warp per (row, token): for the non-anchor tokens of delta rows, replaces scales[row, token]
// (written by row_absmax_kernel, whose values for the anchors are read here) by max|residual|.
template <int DT, int VEC>
__global__ void __launch_bounds__(256) residual_absmax_kernel(const uint16_t *__restrict__ kv, const KvLayout L,
                                                              const float *__restrict__ bins,
                                                              const float *__restrict__ res_bins, int group,
                                                              uint16_t *scales, int row0, int nrows) {
    __shared__ float luts[8][64];
    int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (wid >= static_cast<int64_t>(nrows) * L.ntokens) return;
    wid += static_cast<int64_t>(row0) * L.ntokens;
    const int row = static_cast<int>(wid / L.ntokens), t = static_cast<int>(wid % L.ntokens);
    const int ta = t - t % group;
    const float cqa = half_range(__ldg(bins + row));
    float cqr;
    if (t == ta || !delta_row(res_bins, row, cqa, &cqr)) return;
    float *lut = luts[w];
    lut[lane] = __fdiv_rn(__fsub_rn(static_cast<float>(lane), cqa), cqa);
    lut[lane + 32] = __fdiv_rn(__fsub_rn(static_cast<float>(lane + 32), cqa), cqa);
    __syncwarp();
    const int layer = row % L.nlayers, j = row / L.nlayers;
    const uint16_t *base = kv + layer * L.s_layer + j * L.s_kv;
    const uint16_t *xt = base + t * L.s_token, *xa = base + ta * L.s_token;
    const uint16_t ma_bits = scales[static_cast<int64_t>(row) * L.ntokens + ta];
    const float max_a = Half16<DT>::to_float(ma_bits);
    const float factor_a = __fdiv_rn(cqa, max_a);
    const uint32_t keep = ma_bits ? 0xFFu : 0u;
    uint32_t best = 0;
    if (VEC == 8) {
        const int per_head = L.head_size / 8;
        const int nvec = L.nheads * per_head;
        for (int v = lane; v < nvec; v += 32) {
            const int h = v / per_head, d = (v - h * per_head) * 8;
            const uint4 qt = __ldg(reinterpret_cast<const uint4 *>(xt + h * L.s_head + d));
            const uint4 qa = __ldg(reinterpret_cast<const uint4 *>(xa + h * L.s_head + d));
            const uint32_t wt[4] = {qt.x, qt.y, qt.z, qt.w}, wa[4] = {qa.x, qa.y, qa.z, qa.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint16_t a = static_cast<uint16_t>(wa[e >> 1] >> ((e & 1) * 16));
                const uint16_t x = static_cast<uint16_t>(wt[e >> 1] >> ((e & 1) * 16));
                const uint32_t r = residual_bits<DT>(x, anchor_value<DT>(a, factor_a, cqa, keep, max_a, lut));
                best = max(best, r & 0x7FFFu);
            }
        }
    } else {
        const int C = L.nheads * L.head_size;
        for (int c = lane; c < C; c += 32) {
            const int h = c / L.head_size, d = c - h * L.head_size;
            const uint16_t a = __ldg(xa + h * L.s_head + d), x = __ldg(xt + h * L.s_head + d);
            const uint32_t r = residual_bits<DT>(x, anchor_value<DT>(a, factor_a, cqa, keep, max_a, lut));
            best = max(best, r & 0x7FFFu);
        }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, d));
    if (lane == 0) scales[wid] = static_cast<uint16_t>(best);
}

// Counts to table (normalize_cdf_value, cal_cdf.cu:11-15,40-49), one thread per channel.
// hist: shared uint32 [max_bins+1][kGroup], hist[v][c] = #{sym == v} for v < max_bins; the last row collects
// the symbols outside the table (counted with min(sym, max_bins): no branch), which no entry reads.  Writes the channel's
// lp = max_bins+1 entries to out16 (shared uint16 [kGroup][lp]).
__device__ __forceinline__ void counts_to_table(const uint32_t *hist, int max_bins, int cl, uint16_t *out16) {
    const int lp = max_bins + 1;
    uint32_t total = 0;
    for (int i = 0; i < max_bins; ++i) total += hist[i * kGroup + cl];
    total &= 0xFFFFu;  // the reference accumulates in uint16
    const uint32_t scale = 0xFFFFu - static_cast<uint32_t>(max_bins);
    uint32_t cum = 0;
    for (int i = 0; i <= max_bins; ++i) {
        if (i) cum = (cum + hist[(i - 1) * kGroup + cl]) & 0xFFFFu;
        const uint32_t nv = total ? (scale * cum / total) : 0u;
        out16[cl * lp + i] = static_cast<uint16_t>(nv + i);
    }
}

__device__ __forceinline__ void store_tables(const uint16_t *out16, int16_t *cdf_out, int64_t row, int c0,
                                             int nchannels, int lp, int tid, int nthreads) {
    // the block's tables are one contiguous run of the output
    const int nch = min(kGroup, nchannels - c0);
    uint16_t *dst = reinterpret_cast<uint16_t *>(cdf_out) + (row * nchannels + c0) * lp;
    const int n = nch * lp;
    if (((reinterpret_cast<uintptr_t>(dst) & 3) == 0) && ((n & 1) == 0)) {
        const uint32_t *s32 = reinterpret_cast<const uint32_t *>(out16);
        uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
        for (int i = tid; i < n / 2; i += nthreads) d32[i] = s32[i];
    } else {
        for (int i = tid; i < n; i += nthreads) dst[i] = out16[i];
    }
}

constexpr int kQuantThreads = 256;

// grid (nslab, nrows).  VEC = 8: every thread quantises 8 adjacent channels of one token per step
// (one 128-bit load, one 64-bit symbol store); VEC = 1: scalar fallback for odd shapes.
// DELTA: rows with residual bins (res_bins[row] > 0) quantise every token that is not the first of its
// group of `group` as a residual against its dequantised anchor, with Cq_r = res_bins // 2 - 1 and
// the symbols moved up by Cq_a - Cq_r so that both kinds of token centre on Cq_a.
template <int DT, int VEC, bool DELTA>
__global__ void __launch_bounds__(kQuantThreads) quantize_cdf_kernel(
    const uint16_t *__restrict__ kv, const KvLayout L, const float *__restrict__ bins,
    const uint16_t *__restrict__ scales, int max_bins, int8_t *__restrict__ sym_out,
    int16_t *__restrict__ cdf_out, uint8_t *__restrict__ counts_out, const int64_t *__restrict__ table_row_off,
    int32_t *status, const float *__restrict__ res_bins, int group, int row0) {
    extern __shared__ uint32_t hist[];  // [max_bins+1][kGroup], then uint16 tables [kGroup][lp]
    __shared__ float lut_a[64];
    const int lp = max_bins + 1;
    uint16_t *out16 = reinterpret_cast<uint16_t *>(hist + lp * kGroup);
    const int tid = threadIdx.x;
    const int row = row0 + blockIdx.y, c0 = blockIdx.x * kGroup;
    const int C = L.nheads * L.head_size, T = L.ntokens;
    const int layer = row % L.nlayers, j = row / L.nlayers;
    for (int i = tid; i < lp * kGroup; i += kQuantThreads) hist[i] = 0u;
    __syncthreads();

    const float MAX = half_range(__ldg(bins + row));
    const uint16_t *base = kv + layer * L.s_layer + j * L.s_kv;
    const uint16_t *srow = scales + static_cast<int64_t>(row) * T;
    int8_t *orow = sym_out + static_cast<int64_t>(row) * T * C;
    float cqr = MAX;
    const bool delta = DELTA && delta_row(res_bins, row, MAX, &cqr);
    const uint32_t shift = static_cast<uint32_t>(MAX - cqr);
    if (DELTA) {
        if (tid < 64) lut_a[tid] = __fdiv_rn(__fsub_rn(static_cast<float>(tid), MAX), MAX);
        __syncthreads();
    }

    if (VEC == 8) {
        constexpr int kLanesPerToken = kGroup / 8;                     // 16
        constexpr int kTokensPerStep = kQuantThreads / kLanesPerToken;  // 16
        const int q = tid % kLanesPerToken, tsub = tid / kLanesPerToken;
        const int c = c0 + q * 8;
        const int h = c / L.head_size, d = c - h * L.head_size;
        // lanes q, q+4, q+8, q+12 of a token (and the second token of the warp) start their
        // histogram updates at different channels, so that the 32 lanes of a warp always hit 32
        // different banks of hist[.][channel]
        const int rot = (threadIdx.x & 31) >> 2;
        // for the e-th update of a step: which of the step's eight symbols it counts (a byte selector
        // for the packed pair of words) and the byte offset of that channel inside a histogram row
        uint32_t pick[8], place[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            pick[e] = static_cast<uint32_t>((e + rot) & 7);
            place[e] = static_cast<uint32_t>(q * 8 + ((e + rot) & 7)) * 4u;
        }
        const uint32_t top_bin = static_cast<uint32_t>(max_bins);
        if (c < C) {
            for (int t = tsub; t < T; t += kTokensPerStep) {
                const uint16_t mbits = __ldg(srow + t);
                const bool resid = DELTA && delta && (t % group) != 0;
                const float mq = resid ? cqr : MAX;
                const float factor = __fdiv_rn(mq, Half16<DT>::to_float(mbits));
                const uint32_t keep = mbits ? 0xFFu : 0u;  // all-zero token: 0 * inf = NaN -> symbol 0
                const uint4 x = __ldg(reinterpret_cast<const uint4 *>(base + t * L.s_token + h * L.s_head + d));
                uint32_t w[4] = {x.x, x.y, x.z, x.w};
                if (resid) {  // the token's residuals against its dequantised anchor, in the KV dtype
                    const int ta = t - t % group;
                    const uint16_t ma_bits = __ldg(srow + ta);
                    const float max_a = Half16<DT>::to_float(ma_bits);
                    const float factor_a = __fdiv_rn(MAX, max_a);
                    const uint32_t keep_a = ma_bits ? 0xFFu : 0u;
                    const uint4 xa = __ldg(reinterpret_cast<const uint4 *>(base + ta * L.s_token + h * L.s_head + d));
                    const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const uint32_t lo = residual_bits<DT>(static_cast<uint16_t>(w[e >> 1]),
                                                              anchor_value<DT>(static_cast<uint16_t>(wa[e >> 1]), factor_a, MAX, keep_a, max_a, lut_a));
                        const uint32_t hi = residual_bits<DT>(static_cast<uint16_t>(w[e >> 1] >> 16),
                                                              anchor_value<DT>(static_cast<uint16_t>(wa[e >> 1] >> 16), factor_a, MAX, keep_a, max_a, lut_a));
                        w[e >> 1] = lo | (hi << 16);
                    }
                }
                const uint32_t up = resid ? shift : 0u;
                uint32_t packed[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint16_t hb = static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
                    // three separately rounded fp32 operations, then round-half-even (enc.py:56-57)
                    const float p = __fmul_rn(Half16<DT>::to_float(hb), factor);
                    const float qv = __fadd_rn(p, mq);
                    uint32_t s = __float_as_uint(__fadd_rn(qv, 8388608.0f)) & keep;
                    if (DELTA) s = (s + up) & 0xFFu;
                    packed[e >> 2] |= s << (8 * (e & 3));
                }
                *reinterpret_cast<uint2 *>(orow + static_cast<int64_t>(t) * C + c) = make_uint2(packed[0], packed[1]);
                const char *hist_bytes = reinterpret_cast<const char *>(hist);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t s = __byte_perm(packed[0], packed[1], pick[e]) & 0xFFu;
                    atomicAdd(reinterpret_cast<uint32_t *>(const_cast<char *>(hist_bytes) + min(s, top_bin) * (kGroup * 4u) + place[e]), 1u);
                }
            }
        }
    } else {
        const int cl = tid % kGroup, tsub = tid / kGroup;
        const int c = c0 + cl;
        const int h = c / L.head_size, d = c - h * L.head_size;
        if (c < C) {
            for (int t = tsub; t < T; t += kQuantThreads / kGroup) {
                const uint16_t mbits = __ldg(srow + t);
                const bool resid = DELTA && delta && (t % group) != 0;
                const float mq = resid ? cqr : MAX;
                const float factor = __fdiv_rn(mq, Half16<DT>::to_float(mbits));
                uint16_t hb = __ldg(base + t * L.s_token + h * L.s_head + d);
                if (resid) {
                    const int ta = t - t % group;
                    const uint16_t ma_bits = __ldg(srow + ta);
                    const float max_a = Half16<DT>::to_float(ma_bits);
                    hb = residual_bits<DT>(hb, anchor_value<DT>(__ldg(base + ta * L.s_token + h * L.s_head + d),
                                                                __fdiv_rn(MAX, max_a), MAX, ma_bits ? 0xFFu : 0u, max_a, lut_a));
                }
                const float p = __fmul_rn(Half16<DT>::to_float(hb), factor);
                const float qv = __fadd_rn(p, mq);
                const uint32_t s = ((mbits ? (__float_as_uint(__fadd_rn(qv, 8388608.0f)) & 0xFFu) : 0u) + (resid ? shift : 0u)) & 0xFFu;
                orow[static_cast<int64_t>(t) * C + c] = static_cast<int8_t>(s);
                atomicAdd(&hist[min(s, static_cast<uint32_t>(max_bins)) * kGroup + cl], 1u);
            }
        }
    }
    __syncthreads();
    if (tid < kGroup && c0 + tid < C) counts_to_table(hist, max_bins, tid, out16);
    if (counts_out) {
        // byte counts of the non-centre symbols, [symbol][channel] so that a warp writes a run of bytes
        const int cq = static_cast<int>(MAX);
        uint8_t *dst = counts_out + __ldg(table_row_off + row) + c0;
        bool overflow = false;
        for (int i = tid; i < 2 * cq * kGroup; i += kQuantThreads) {
            const int jj = i / kGroup, cl = i - jj * kGroup;
            const int sym = jj < cq ? jj : jj + 1;
            const uint32_t n = (sym < max_bins) ? hist[sym * kGroup + cl] : 0u;
            if (c0 + cl < C) {
                dst[static_cast<int64_t>(jj) * C + cl] = static_cast<uint8_t>(n);
                overflow |= n > 255u;
            }
        }
        // a symbol above 2*Cq (which the quantiser never produces) has no place in the byte counts
        for (int i = tid; i < (max_bins - 2 * cq - 1) * kGroup; i += kQuantThreads) {
            const int sym = 2 * cq + 1 + i / kGroup, cl = i % kGroup;
            overflow |= (c0 + cl < C) && hist[sym * kGroup + cl] != 0u;
        }
        if (overflow && status) atomicOr(status, CG_S_COUNT_OVERFLOW);
    }
    __syncthreads();
    store_tables(out16, cdf_out, row, c0, C, lp, tid, kQuantThreads);
}

// calculate_cdf on int8 symbols with arbitrary strides: grid (nslab, nrows), 256 threads, thread
// (channel = tid % 128, token parity = tid / 128).
__global__ void __launch_bounds__(kQuantThreads) symbol_cdf_kernel(const int8_t *__restrict__ sym, int64_t s0,
                                                                   int64_t s1, int64_t s2, int ntokens,
                                                                   int nchannels, int max_bins,
                                                                   int16_t *__restrict__ cdf_out) {
    extern __shared__ uint32_t hist[];
    const int lp = max_bins + 1;
    uint16_t *out16 = reinterpret_cast<uint16_t *>(hist + lp * kGroup);
    const int tid = threadIdx.x, cl = tid % kGroup, tsub = tid / kGroup;
    const int row = blockIdx.y, c0 = blockIdx.x * kGroup, c = c0 + cl;
    for (int i = tid; i < lp * kGroup; i += kQuantThreads) hist[i] = 0u;
    __syncthreads();
    if (c < nchannels) {
        const int8_t *p = sym + row * s0 + c * s2;
        for (int t = tsub; t < ntokens; t += kQuantThreads / kGroup) {
            const uint32_t s = static_cast<uint8_t>(__ldg(p + t * s1));
            atomicAdd(&hist[min(s, static_cast<uint32_t>(max_bins)) * kGroup + cl], 1u);
        }
    }
    __syncthreads();
    if (tid < kGroup && c < nchannels) counts_to_table(hist, max_bins, tid, out16);
    __syncthreads();
    store_tables(out16, cdf_out, row, c0, nchannels, lp, tid, kQuantThreads);
}

static size_t hist_smem_bytes(int max_bins) {
    const int lp = max_bins + 1;
    return static_cast<size_t>(lp) * kGroup * 4 + static_cast<size_t>(lp) * kGroup * 2;
}

}  // namespace cg

using namespace cg;

extern "C" int cg_calculate_cdf(const int8_t *sym, const int64_t sym_strides[3], int nrows, int ntokens,
                                int nchannels, int max_bins, int16_t *cdf_out, void *stream) {
    if (!sym || !sym_strides || !cdf_out) return CG_E_NULL;
    if (nrows <= 0 || ntokens <= 0 || nchannels <= 0 || nrows > 65535) return CG_E_SHAPE;
    if (max_bins < 1 || max_bins >= CG_MAX_LP) return CG_E_LP;
    if (ntokens >= 65536) return CG_E_HIST;
    const dim3 grid((nchannels + kGroup - 1) / kGroup, nrows);
    symbol_cdf_kernel<<<grid, kQuantThreads, hist_smem_bytes(max_bins), static_cast<cudaStream_t>(stream)>>>(
        sym, sym_strides[0], sym_strides[1], sym_strides[2], ntokens, nchannels, max_bins, cdf_out);
    return check_launch();
}

namespace {

struct QuantShape {
    KvLayout L;
    bool vec;
};

// argument checks shared by the quantise entry points
int quant_shape(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token, int64_t s_head,
                int nlayers, int ntokens, int nheads, int head_size, const void *sym_out, QuantShape *q) {
    if (nlayers <= 0 || ntokens <= 0 || nheads <= 0 || head_size <= 0 || 2 * nlayers > 65535) return CG_E_SHAPE;
    if (ntokens >= 65536) return CG_E_HIST;
    if (dtype != CG_F16 && dtype != CG_BF16) return CG_E_DTYPE;
    q->L = KvLayout{s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size};
    // the 128-bit path needs 8-channel runs that stay inside one head and 16-byte aligned rows
    q->vec = (head_size % 8 == 0) && ((reinterpret_cast<uintptr_t>(kv) & 15) == 0) && (s_layer % 8 == 0) &&
             (s_kv % 8 == 0) && (s_token % 8 == 0) && (s_head % 8 == 0) &&
             ((reinterpret_cast<uintptr_t>(sym_out) & 7) == 0);
    return CG_OK;
}

// Rows of one window of the quantise passes.  Windows small enough for the 126 MB L2 would let the
// quantise pass find the KV that the max|x| pass just read, but measured on a 256-token Llama-7B chunk
// (134 MB of KV, three windows) the smaller launches cost more than the second read from HBM does:
// 0.60 ms against 0.54 ms for the whole encode.  So one window: all rows.
int window_rows(const QuantShape &q) { return 2 * q.L.nlayers; }

int launch_absmax(const uint16_t *x, const QuantShape &q, uint16_t *sc, cudaStream_t st, int row0 = 0, int nrows = -1) {
    if (nrows < 0) nrows = 2 * q.L.nlayers;
    const int64_t nwarps = static_cast<int64_t>(nrows) * q.L.ntokens;
    const unsigned ablocks = static_cast<unsigned>((nwarps * 32 + 255) / 256);
    if (q.vec) row_absmax_kernel<8><<<ablocks, 256, 0, st>>>(x, q.L, sc, row0, nrows);
    else row_absmax_kernel<1><<<ablocks, 256, 0, st>>>(x, q.L, sc, row0, nrows);
    return check_launch();
}

int launch_quantize(const uint16_t *x, int dtype, const QuantShape &q, const float *bins, const uint16_t *sc,
                    int max_bins, int8_t *sym_out, int16_t *cdf_out, uint8_t *counts_out,
                    const int64_t *table_row_off, int32_t *status, cudaStream_t st, const float *res_bins = nullptr,
                    int group = 0, int row0 = 0, int nrows = -1) {
    if (nrows < 0) nrows = 2 * q.L.nlayers;
    const int C = q.L.nheads * q.L.head_size;
    const dim3 grid((C + kGroup - 1) / kGroup, nrows);
    const size_t smem = hist_smem_bytes(max_bins);
#define CG_LAUNCH_Q(DT, V, D) \
    quantize_cdf_kernel<DT, V, D><<<grid, kQuantThreads, smem, st>>>(x, q.L, bins, sc, max_bins, sym_out, cdf_out, \
                                                                     counts_out, table_row_off, status, res_bins, group, row0)
    if (group > 0) {
        if (dtype == CG_F16) { if (q.vec) CG_LAUNCH_Q(CG_F16, 8, true); else CG_LAUNCH_Q(CG_F16, 1, true); }
        else { if (q.vec) CG_LAUNCH_Q(CG_BF16, 8, true); else CG_LAUNCH_Q(CG_BF16, 1, true); }
    } else {
        if (dtype == CG_F16) { if (q.vec) CG_LAUNCH_Q(CG_F16, 8, false); else CG_LAUNCH_Q(CG_F16, 1, false); }
        else { if (q.vec) CG_LAUNCH_Q(CG_BF16, 8, false); else CG_LAUNCH_Q(CG_BF16, 1, false); }
    }
#undef CG_LAUNCH_Q
    return check_launch();
}

int launch_residual_absmax(const uint16_t *x, int dtype, const QuantShape &q, const float *bins,
                           const float *res_bins, int group, uint16_t *sc, cudaStream_t st, int row0, int nrows) {
    const int64_t nwarps = static_cast<int64_t>(nrows) * q.L.ntokens;
    const unsigned blocks = static_cast<unsigned>((nwarps * 32 + 255) / 256);
    if (dtype == CG_F16) {
        if (q.vec) residual_absmax_kernel<CG_F16, 8><<<blocks, 256, 0, st>>>(x, q.L, bins, res_bins, group, sc, row0, nrows);
        else residual_absmax_kernel<CG_F16, 1><<<blocks, 256, 0, st>>>(x, q.L, bins, res_bins, group, sc, row0, nrows);
    } else {
        if (q.vec) residual_absmax_kernel<CG_BF16, 8><<<blocks, 256, 0, st>>>(x, q.L, bins, res_bins, group, sc, row0, nrows);
        else residual_absmax_kernel<CG_BF16, 1><<<blocks, 256, 0, st>>>(x, q.L, bins, res_bins, group, sc, row0, nrows);
    }
    return check_launch();
}

}  // namespace

extern "C" int cg_row_absmax(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                             int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                             void *scales_out, void *stream) {
    if (!kv || !scales_out) return CG_E_NULL;
    QuantShape q;
    // the symbol pointer only matters for the quantise pass: any 8-byte aligned value keeps the choice of load width
    if (int rc = quant_shape(kv, dtype, s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size, nullptr, &q))
        return rc;
    return launch_absmax(static_cast<const uint16_t *>(kv), q, static_cast<uint16_t *>(scales_out),
                         static_cast<cudaStream_t>(stream));
}

extern "C" int cg_quantize_cdf_scaled(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                                      int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                                      const float *bins, int max_bins, const void *scales, int8_t *sym_out,
                                      int16_t *cdf_out, uint8_t *counts_out, const int64_t *table_row_off,
                                      int32_t *status, void *stream) {
    if (!kv || !bins || !sym_out || !scales || !cdf_out) return CG_E_NULL;
    if (counts_out && !table_row_off) return CG_E_NULL;
    if (max_bins < 1 || max_bins >= CG_MAX_LP) return CG_E_LP;
    QuantShape q;
    if (int rc = quant_shape(kv, dtype, s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size, sym_out, &q))
        return rc;
    return launch_quantize(static_cast<const uint16_t *>(kv), dtype, q, bins, static_cast<const uint16_t *>(scales),
                           max_bins, sym_out, cdf_out, counts_out, table_row_off, status,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int cg_quantize_cdf(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                               int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                               const float *bins, int max_bins, int8_t *sym_out, void *scales_out,
                               int16_t *cdf_out, uint8_t *counts_out, const int64_t *table_row_off,
                               int32_t *status, void *stream) {
    if (!kv || !bins || !sym_out || !scales_out || !cdf_out) return CG_E_NULL;
    if (counts_out && !table_row_off) return CG_E_NULL;
    if (nlayers <= 0 || ntokens <= 0 || nheads <= 0 || head_size <= 0 || 2 * nlayers > 65535) return CG_E_SHAPE;
    if (max_bins < 1 || max_bins >= CG_MAX_LP) return CG_E_LP;
    QuantShape q;
    if (int rc = quant_shape(kv, dtype, s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size, sym_out, &q))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t *x = static_cast<const uint16_t *>(kv);
    uint16_t *sc = static_cast<uint16_t *>(scales_out);
    const int total = 2 * nlayers, step = window_rows(q);
    for (int r0 = 0; r0 < total; r0 += step) {
        const int n = total - r0 < step ? total - r0 : step;
        if (int rc = launch_absmax(x, q, sc, st, r0, n)) return rc;
        if (int rc = launch_quantize(x, dtype, q, bins, sc, max_bins, sym_out, cdf_out, counts_out, table_row_off,
                                     status, st, nullptr, 0, r0, n))
            return rc;
    }
    return CG_OK;
}

extern "C" int cg_quantize_cdf_delta(const void *kv, int dtype, int64_t s_layer, int64_t s_kv, int64_t s_token,
                                     int64_t s_head, int nlayers, int ntokens, int nheads, int head_size,
                                     const float *bins, int max_bins, int delta_group, const float *res_bins,
                                     int8_t *sym_out, void *scales_out, int16_t *cdf_out, uint8_t *counts_out,
                                     const int64_t *table_row_off, int32_t *status, void *stream) {
    if (delta_group == 0)
        return cg_quantize_cdf(kv, dtype, s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size, bins,
                               max_bins, sym_out, scales_out, cdf_out, counts_out, table_row_off, status, stream);
    if (!kv || !bins || !res_bins || !sym_out || !scales_out || !cdf_out) return CG_E_NULL;
    if (counts_out && !table_row_off) return CG_E_NULL;
    if (delta_group < 2 || delta_group > CG_MAX_TOKENS_PER_STREAM || CG_MAX_TOKENS_PER_STREAM % delta_group)
        return CG_E_SHAPE;
    if (max_bins < 1 || max_bins >= CG_MAX_LP) return CG_E_LP;
    QuantShape q;
    if (int rc = quant_shape(kv, dtype, s_layer, s_kv, s_token, s_head, nlayers, ntokens, nheads, head_size, sym_out, &q))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t *x = static_cast<const uint16_t *>(kv);
    uint16_t *sc = static_cast<uint16_t *>(scales_out);
    const int total = 2 * nlayers, step = window_rows(q);
    for (int r0 = 0; r0 < total; r0 += step) {
        const int n = total - r0 < step ? total - r0 : step;
        if (int rc = launch_absmax(x, q, sc, st, r0, n)) return rc;
        if (int rc = launch_residual_absmax(x, dtype, q, bins, res_bins, delta_group, sc, st, r0, n)) return rc;
        if (int rc = launch_quantize(x, dtype, q, bins, sc, max_bins, sym_out, cdf_out, counts_out, table_row_off,
                                     status, st, res_bins, delta_group, r0, n))
            return rc;
    }
    return CG_OK;
}
