// Arithmetic encoder kernels: one thread per stream, 128 adjacent channels of one row per block,
// every sub-chunk of a chunk in one launch; then offsets by a two-level scan and a gather.
//
// The per-symbol step lives in cg_coder.cuh.
#include "cg_common.cuh"

namespace cg {

struct EncodeParams {
    const int16_t *cdf;  // [nrows, C, lp]
    const int8_t *sym;   // element (row, token, channel) at sym[row*s0 + token*s1 + channel*s2]
    int64_t s0, s1, s2;
    int ntokens, nchannels, lp;
    uint8_t *scratch;     // [nsub, nrows*C, stride]
    int64_t stride;
    int32_t *lengths;     // [nsub, nrows*C]
    int32_t *status;
};

// see EncoderState::add_f
__constant__ uint32_t opaque_one = 1u;
__constant__ uint32_t opaque_minus_one = 0xFFFFFFFFu;

constexpr int kPrefetch = 8;  // symbols fetched ahead of the coder

__global__ void __launch_bounds__(kGroup) encode_kernel(const EncodeParams p) {
    extern __shared__ uint32_t tab[];
    const int tid = threadIdx.x;
    const int row = blockIdx.y, sub = blockIdx.z;
    const int c = blockIdx.x * kGroup + tid;
    // the lanes that encode together, taken while the warp is still converged
    const uint32_t lanes = __ballot_sync(0xFFFFFFFFu, c < p.nchannels);
    if (c >= p.nchannels) return;  // no block barrier in this kernel
    const int nrows = gridDim.y;
    const int64_t g = static_cast<int64_t>(row) * p.nchannels + c;
    const int t0 = sub * kSubTokens;
    const int n = min(kSubTokens, p.ntokens - t0);
    const int maxsym = p.lp - 2;

    stage_table_column(tab, p.cdf + g * p.lp, p.lp, p.lp, tid);
    const uint32_t col = smem_addr(tab + tid);
    const int64_t slot = static_cast<int64_t>(sub) * nrows * p.nchannels + g;
    BitSink out;
    out.init(p.scratch + slot * p.stride, p.stride);

    const int8_t *sp = p.sym + row * p.s0 + static_cast<int64_t>(t0) * p.s1 + c * p.s2;
    EncoderState enc;
    enc.init(opaque_one, opaque_minus_one);
    uint32_t largest = 0;  // the largest symbol met: one above maxsym is reported and coded as maxsym

    // whole groups of kPrefetch symbols: their loads are issued together, ahead of the coder, with no
    // bound checks; the last, shorter group goes symbol by symbol
    const int64_t s1 = p.s1;
    const uint8_t *sp8 = reinterpret_cast<const uint8_t *>(sp);
    const uint32_t top = static_cast<uint32_t>(maxsym);
    int base = 0;
    for (; base + kPrefetch <= n; base += kPrefetch) {
        uint32_t buf[kPrefetch];
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) buf[j] = __ldg(sp8 + j * s1);
        sp8 += kPrefetch * s1;
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) {
            largest = max(largest, buf[j]);
            enc.step(Smem{}, col, min(buf[j], top), top, out, lanes);
        }
    }
    for (; base < n; ++base) {
        const uint32_t s = __ldg(sp8);
        sp8 += s1;
        largest = max(largest, s);
        enc.step(Smem{}, col, min(s, top), top, out, lanes);
    }
    const uint32_t nbytes = enc.flush(out);
    p.lengths[slot] = static_cast<int32_t>(nbytes);
    if (p.status) {
        int bits = 0;
        if (static_cast<int64_t>(nbytes) > p.stride) bits |= CG_S_STREAM_OVERFLOW;
        if (largest > static_cast<uint32_t>(maxsym)) bits |= CG_S_BAD_SYMBOL;
        if (bits) atomicOr(p.status, bits);
    }
}

// ---- offsets --------------------------------------------------------------------------------------------
// Segments are either the sub-chunks of one encode call (flat lengths array [nseg, nrows*C]) or the
// jobs of one decode call (one lengths pointer and one expected byte total per job).
struct SegmentList {
    const void *lengths[CG_MAX_DECODE_JOBS];
    int64_t expect[CG_MAX_DECODE_JOBS];
    int32_t kind[CG_MAX_DECODE_JOBS];  // CG_LENGTHS_*
};

// Level 1: one warp per 128-channel group sums the group's lengths into sums[nseg, nrows*nslab].
template <bool BY_JOB>
__global__ void group_sums_kernel(const __grid_constant__ SegmentList segs, const int32_t *flat_lengths,
                                  int nseg, int nrows, int nchannels, int nslab, int64_t *sums,
                                  int32_t *status) {
    const int ngroups = nrows * nslab;
    const int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<int64_t>(nseg) * ngroups) return;
    const int seg = static_cast<int>(wid / ngroups), gid = static_cast<int>(wid % ngroups);
    const int row = gid / nslab, slab = gid % nslab;
    const bool u16 = BY_JOB && segs.kind[seg] == CG_LENGTHS_U16;
    const int32_t *len = BY_JOB ? static_cast<const int32_t *>(segs.lengths[seg])
                                : flat_lengths + static_cast<int64_t>(seg) * nrows * nchannels;
    const uint16_t *len16 = reinterpret_cast<const uint16_t *>(len) + static_cast<int64_t>(row) * nchannels;
    len += static_cast<int64_t>(row) * nchannels;
    int64_t s = 0;
    bool bad = false;
    for (int c = slab * kGroup + lane; c < min(nchannels, (slab + 1) * kGroup); c += 32) {
        int v = u16 ? static_cast<int>(__ldg(len16 + c)) : __ldg(len + c);
        if (v < 0) { v = 0; bad = true; }
        if (v > (1 << 20)) { v = 1 << 20; bad = true; }
        s += v;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, d);
    if (lane == 0) sums[wid] = s;
    if (bad && status) atomicOr(status, CG_S_BAD_LENGTHS);
}

// Level 2: one block per segment turns its group sums into exclusive offsets, in place.  The
// segment total goes to totals[seg] (encode) or is compared with the job's byte count (decode).
constexpr int kScanThreads = 1024;
template <bool BY_JOB>
__global__ void __launch_bounds__(kScanThreads) group_scan_kernel(const __grid_constant__ SegmentList segs,
                                                                   int64_t *sums, int ngroups,
                                                                   int64_t *totals, int32_t *status) {
    __shared__ int64_t part[kScanThreads];
    const int seg = blockIdx.x, tid = threadIdx.x;
    int64_t *s = sums + static_cast<int64_t>(seg) * ngroups;
    const int per = (ngroups + kScanThreads - 1) / kScanThreads;
    const int b = min(ngroups, tid * per), e = min(ngroups, b + per);
    int64_t local = 0;
    for (int i = b; i < e; ++i) local += s[i];
    part[tid] = local;
    __syncthreads();
    for (int d = 1; d < kScanThreads; d <<= 1) {  // Hillis-Steele inclusive scan of the partials
        const int64_t v = (tid >= d) ? part[tid - d] : 0;
        __syncthreads();
        part[tid] += v;
        __syncthreads();
    }
    int64_t run = part[tid] - local;
    for (int i = b; i < e; ++i) {
        const int64_t v = s[i];
        s[i] = run;
        run += v;
    }
    if (tid == kScanThreads - 1) {
        const int64_t total = part[tid];
        if (!BY_JOB) totals[seg] = total;
        if (BY_JOB && segs.expect[seg] != total && status) atomicOr(status, CG_S_BAD_LENGTHS);
    }
}

// Exclusive scan of the nsub segment totals into sub_off[0..nsub] (one warp, serial in chunks of 32).
__global__ void segment_offsets_kernel(const int64_t *totals, int nsub, int64_t *sub_off) {
    const int lane = threadIdx.x;
    int64_t carry = 0;
    for (int b = 0; b < nsub; b += 32) {
        const int64_t v = (b + lane < nsub) ? totals[b + lane] : 0;
        int64_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int64_t n = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += n;
        }
        if (b + lane < nsub) sub_off[b + lane] = carry + incl - v;
        carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (lane == 0) sub_off[nsub] = carry;
}

// ---- gather (second half of collect_bytes, cachegen_encoder.py:210-222) ------------------------------------
// One block per (group, row, sub-chunk).  Eight lanes copy one stream: its scratch row is read as
// aligned 32-bit words (one per lane and step) and written byte by byte to where the stream goes
// (streams lie back to back, so the destination has no alignment); a warp has four streams in flight
// and a block sixteen, which is what hides the latency of these short dependent copies.
__global__ void __launch_bounds__(kGroup) compact_kernel(const uint8_t *scratch, int64_t stride,
                                                         const int32_t *lengths, const int64_t *group_off,
                                                         const int64_t *sub_off, int nchannels,
                                                         uint8_t *bytes_out) {
    __shared__ int warp_sums[kGroup / 32];
    __shared__ int offs[kGroup];
    __shared__ int lens[kGroup];
    const int tid = threadIdx.x;
    const int row = blockIdx.y, sub = blockIdx.z, nrows = gridDim.y, nslab = gridDim.x;
    const int c = blockIdx.x * kGroup + tid;
    const int64_t slot0 = (static_cast<int64_t>(sub) * nrows + row) * nchannels + blockIdx.x * kGroup;
    const int len = (c < nchannels) ? lengths[slot0 + tid] : 0;
    const int excl = block_exclusive_scan_128(len, warp_sums, tid, nullptr);
    offs[tid] = excl;
    lens[tid] = len;
    __syncthreads();
    const int64_t gid = (static_cast<int64_t>(sub) * nrows + row) * nslab + blockIdx.x;
    uint8_t *dst0 = bytes_out + sub_off[sub] + group_off[gid];
    constexpr int kLanesPerStream = 8;
    const int part = tid % kLanesPerStream;
    for (int s = tid / kLanesPerStream; s < kGroup; s += kGroup / kLanesPerStream) {
        const int n = min(lens[s], static_cast<int>(stride));  // a longer stream was truncated and reported by the encoder
        const uint32_t *src = reinterpret_cast<const uint32_t *>(scratch + (slot0 + s) * stride);
        uint8_t *dst = dst0 + offs[s];
        for (int j = part * 4; j < n; j += kLanesPerStream * 4) {
            const uint32_t w = __ldg(src + (j >> 2));
            dst[j] = static_cast<uint8_t>(w);
            if (j + 1 < n) dst[j + 1] = static_cast<uint8_t>(w >> 8);
            if (j + 2 < n) dst[j + 2] = static_cast<uint8_t>(w >> 16);
            if (j + 3 < n) dst[j + 3] = static_cast<uint8_t>(w >> 24);
        }
    }
}

}  // namespace cg

using namespace cg;

static int launch_encode(const EncodeParams &p, int nrows, int nsub, cudaStream_t st) {
    const dim3 grid((p.nchannels + kGroup - 1) / kGroup, nrows, nsub);
    const size_t smem = static_cast<size_t>(p.lp) * kRowBytes;
    encode_kernel<<<grid, kGroup, smem, st>>>(p);
    return check_launch();
}

extern "C" int cg_encode_padded(const int16_t *cdf, const int8_t *sym, const int64_t sym_strides[3],
                                int nrows, int ntokens, int nchannels, int lp, uint8_t *out_buf,
                                int64_t out_stride, int32_t *out_lengths, int32_t *status, void *stream) {
    if (!cdf || !sym || !sym_strides || !out_buf || !out_lengths) return CG_E_NULL;
    if (nrows <= 0 || ntokens <= 0 || nchannels <= 0 || nrows > 65535) return CG_E_SHAPE;
    if (ntokens > CG_MAX_TOKENS_PER_STREAM) return CG_E_TOKENS;
    if (lp < 2 || lp > CG_MAX_LP) return CG_E_LP;
    if (out_stride < 4 || (out_stride & 3) || (reinterpret_cast<uintptr_t>(out_buf) & 3)) return CG_E_ALIGN;
    EncodeParams p{cdf, sym, sym_strides[0], sym_strides[1], sym_strides[2], ntokens, nchannels, lp,
                   out_buf, out_stride, out_lengths, status};
    return launch_encode(p, nrows, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int cg_encode_chunk(const int16_t *cdf, const int8_t *sym, int nrows, int ntokens,
                               int nchannels, int lp, uint8_t *scratch, int64_t scratch_stride,
                               int32_t *lengths_out, int64_t *group_off_out, int64_t *sub_off_out,
                               int32_t *status, void *stream) {
    if (!cdf || !sym || !scratch || !lengths_out || !group_off_out || !sub_off_out) return CG_E_NULL;
    if (nrows <= 0 || ntokens <= 0 || nchannels <= 0 || nrows > 65535) return CG_E_SHAPE;
    if (lp < 2 || lp > CG_MAX_LP) return CG_E_LP;
    if (scratch_stride < 4 || (scratch_stride & 3) || (reinterpret_cast<uintptr_t>(scratch) & 3)) return CG_E_ALIGN;
    const int nsub = (ntokens + kSubTokens - 1) / kSubTokens;
    if (nsub > 65535) return CG_E_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    EncodeParams p{cdf, sym, static_cast<int64_t>(ntokens) * nchannels, nchannels, 1, ntokens, nchannels, lp,
                   scratch, scratch_stride, lengths_out, status};
    if (int rc = launch_encode(p, nrows, nsub, st)) return rc;
    const int nslab = (nchannels + kGroup - 1) / kGroup;
    const int ngroups = nrows * nslab;
    const int64_t nwarps = static_cast<int64_t>(nsub) * ngroups;
    SegmentList none{};
    group_sums_kernel<false><<<static_cast<unsigned>((nwarps * 32 + 255) / 256), 256, 0, st>>>(
        none, lengths_out, nsub, nrows, nchannels, nslab, group_off_out, status);
    if (int rc = check_launch()) return rc;
    // the segment totals are parked in sub_off_out[1..nsub] and scanned in place afterwards
    group_scan_kernel<false><<<nsub, kScanThreads, 0, st>>>(none, group_off_out, ngroups, sub_off_out + 1, status);
    if (int rc = check_launch()) return rc;
    segment_offsets_kernel<<<1, 32, 0, st>>>(sub_off_out + 1, nsub, sub_off_out);
    return check_launch();
}

extern "C" int cg_compact_streams(const uint8_t *scratch, int64_t scratch_stride, const int32_t *lengths,
                                  const int64_t *group_off, const int64_t *sub_off, int nsub, int nrows,
                                  int nchannels, uint8_t *bytes_out, void *stream) {
    if (!scratch || !lengths || !group_off || !sub_off || !bytes_out) return CG_E_NULL;
    if (nsub <= 0 || nrows <= 0 || nchannels <= 0 || nrows > 65535 || nsub > 65535) return CG_E_SHAPE;
    // the rows are read as 32-bit words, as cg_encode_chunk wrote them
    if (scratch_stride < 4 || (scratch_stride & 3) || (reinterpret_cast<uintptr_t>(scratch) & 3)) return CG_E_ALIGN;
    const dim3 grid((nchannels + kGroup - 1) / kGroup, nrows, nsub);
    compact_kernel<<<grid, kGroup, 0, static_cast<cudaStream_t>(stream)>>>(scratch, scratch_stride, lengths,
                                                                          group_off, sub_off, nchannels, bytes_out);
    return check_launch();
}

// ---- offsets for the decode side (shares the scan kernels) -------------------------------------------------
extern "C" int cg_decode_offsets(const cg_decode_job *jobs_host, int njobs, int nrows, int nchannels,
                                 int64_t *group_off_out, int32_t *status, void *stream) {
    if (!jobs_host || !group_off_out) return CG_E_NULL;
    if (njobs <= 0 || nrows <= 0 || nchannels <= 0) return CG_E_SHAPE;
    if (njobs > CG_MAX_DECODE_JOBS) return CG_E_CAPACITY;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SegmentList segs;
    for (int j = 0; j < njobs; ++j) {
        if (!jobs_host[j].lengths) return CG_E_NULL;
        segs.lengths[j] = jobs_host[j].lengths;
        segs.expect[j] = jobs_host[j].nbytes;
        segs.kind[j] = jobs_host[j].length_kind;
    }
    const int nslab = (nchannels + kGroup - 1) / kGroup;
    const int ngroups = nrows * nslab;
    const int64_t nwarps = static_cast<int64_t>(njobs) * ngroups;
    group_sums_kernel<true><<<static_cast<unsigned>((nwarps * 32 + 255) / 256), 256, 0, st>>>(
        segs, nullptr, njobs, nrows, nchannels, nslab, group_off_out, status);
    if (int rc = check_launch()) return rc;
    group_scan_kernel<true><<<njobs, kScanThreads, 0, st>>>(segs, group_off_out, ngroups, nullptr, status);
    return check_launch();
}
