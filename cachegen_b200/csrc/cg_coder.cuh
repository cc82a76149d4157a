// The per-stream arithmetic coder: bit window, bit sink, decode loop and encode step.
//
// This header compiles both as CUDA device code (the product) and as plain host C++ (only so that
// the CPU test-suite can drive exactly these loops against the oracle without a GPU; the shared
// library never contains or calls a host build of them).
//
// The steps restate the reference's loops
// (LMCache/third_party/torchac_cuda/torchac_kernel_dec_new.cu:262-302 and
//  torchac_kernel_enc_new.cu:255-306) without the 64-bit division, the binary search on `count`
// and the bit-serial renormalisation:
//   * cdf[m] <= count, count = ((value-low+1)*2^16 - 1) / span, holds exactly when
//     (span*cdf[m]) >> 16 <= value - low, so the search compares scaled table entries with
//     value - low directly;
//   * within one symbol the renormalisation loop does a run of "equal top bit" shifts followed
//     by a run of "underflow" shifts, never the other way round; both run lengths come from a
//     count-leading-zeros, the decoder takes all its new bits in one funnel shift and the encoder
//     emits the shifted-out top bits of `low` in one append.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define CG_HD __host__ __device__ __forceinline__
#else
#define CG_HD inline
#endif

namespace cg {

constexpr int kGroupChannels = 128;            // streams (threads) per coder block
constexpr int kTableRowBytes = kGroupChannels * 4;  // bytes between table entries m and m+1 of a stream

// ---- intrinsics with host stand-ins -----------------------------------------------------------------
CG_HD int cg_clz(uint32_t x) {
#if defined(__CUDA_ARCH__)
    return __clz(static_cast<int>(x));
#else
    return x ? __builtin_clz(x) : 32;
#endif
}
// upper 32 bits of (hi:lo) << (s & 31)
CG_HD uint32_t cg_fshl(uint32_t lo, uint32_t hi, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_l(lo, hi, s);
#else
    s &= 31u;
    return s ? ((hi << s) | (lo >> (32u - s))) : hi;
#endif
}
// upper 32 bits of (hi:lo) << min(s, 32)
CG_HD uint32_t cg_fshl_clamp(uint32_t lo, uint32_t hi, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_lc(lo, hi, s);
#else
    if (s >= 32u) return lo;
    return s ? ((hi << s) | (lo >> (32u - s))) : hi;
#endif
}
// lower 32 bits of (hi:lo) >> min(s, 32)
CG_HD uint32_t cg_fshr_clamp(uint32_t lo, uint32_t hi, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_rc(lo, hi, s);
#else
    if (s >= 32u) return hi;
    return s ? ((lo >> s) | (hi << (32u - s))) : lo;
#endif
}
CG_HD uint32_t cg_bswap32(uint32_t v) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(v, 0, 0x0123);
#else
    return __builtin_bswap32(v);
#endif
}
CG_HD uint32_t cg_load_stream_word(const uint32_t *p) {
#if defined(__CUDA_ARCH__)
    return __ldg(p);
#else
    return *p;
#endif
}

// upper 32 bits of span * c16 where span = spanm1 + 1 (span may be 2^32) and c16 = cdf << 16:
// equals the (span * cdf) >> 16 of the range update (enc_new.cu:262-263), without the 64-bit shift.
CG_HD uint32_t scale_by_cdf(uint32_t spanm1, uint32_t c16) {
    const uint64_t t = static_cast<uint64_t>(spanm1) * c16 + c16;
    return static_cast<uint32_t>(t >> 32);
}

// Count of equal-top-bit shifts for the interval [low, high] (the |1 keeps it below 32 on a
// degenerate interval, which only a corrupt table can produce).
CG_HD int equal_shifts(uint32_t low, uint32_t high) { return cg_clz((low ^ high) | 1u); }
// Count of underflow shifts once the top bits differ: the run, from bit 30 down, of positions where
// low has a 1 and high a 0.
CG_HD int underflow_shifts(uint32_t low, uint32_t high) { return cg_clz((((~low) | high) << 1) | 1u); }

// ---- shared-memory access --------------------------------------------------------------------------------
// A stream's table is the column tab[m][tid] = cdf[m] << 16 of a [rows][128] uint32 array, addressed
// by byte address: entry m of the column starting at `col` is at col + m * kTableRowBytes.  The
// stream's bit ring (below) is a column of the same shape.  On the device the addresses are
// shared-memory addresses (bank = lane for every row); on the host they are offsets into a plain array.
struct Smem {
#if defined(__CUDA_ARCH__)
    __device__ __forceinline__ uint32_t ld(uint32_t addr) const {
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
        return v;
    }
    __device__ __forceinline__ void st(uint32_t addr, uint32_t v) const {
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
    }
#else
    uint8_t *base;
    uint32_t ld(uint32_t addr) const { return *reinterpret_cast<const uint32_t *>(base + addr); }
    void st(uint32_t addr, uint32_t v) const { *reinterpret_cast<uint32_t *>(base + addr) = v; }
#endif
};

// ---- MSB-first bit ring over one stream --------------------------------------------------------------
// Each thread keeps the next 128 bytes of its stream in a column of shared memory, 32 rows of one
// big-endian 32-bit word plus a 33rd row that repeats row 0's newest word, so that the two words under
// any bit position are at [row] and [row + 1] without a wrap test.  The per-symbol read is branch-free;
// a stream longer than the ring is topped up 16 words at a time once the reader has left the half that
// is overwritten (0.3 % of the streams of the benchmark workload are longer than 128 bytes).
//
// The byte array is read as aligned 32-bit words; bits before the stream's first byte are skipped by
// the start position and words (or word tails) past its last byte are stored as zero, which is what
// the reference sees in its zero-padded staging row (dec_new.cu:229-232).
constexpr int kRingWords = 32;
constexpr int kRingRows = kRingWords + 1;

struct BitRing {
    const uint32_t *wp;    // word holding the stream's first byte
    uint32_t end_bit;      // bit index, counted from wp, one past the stream's last bit
    uint32_t ring;         // address of this stream's ring column (row 0)
    uint32_t pos;          // bit index, counted from wp, of the next unread bit
    uint32_t next_refill;  // reaching this position triggers a top-up
    uint32_t loaded;       // stream words placed in the ring so far

    CG_HD uint32_t fetch(uint32_t j) const {
        const uint32_t b0 = j * 32u;
        if (b0 >= end_bit) return 0u;
        uint32_t w = cg_bswap32(cg_load_stream_word(wp + j));
        const uint32_t rem = end_bit - b0;
        if (rem < 32u) w &= 0xFFFFFFFFu << (32u - rem);
        return w;
    }
    // the 32 bits at the current position
    CG_HD uint32_t peek(Smem sm) const {
        const uint32_t a = ring + ((pos << 4) & (static_cast<uint32_t>(kRingWords - 1) * kTableRowBytes));
        return cg_fshl(sm.ld(a + kTableRowBytes), sm.ld(a), pos);
    }
    // fills the ring; returns the stream's first 32 bits (the coder's initial `value`, dec_new.cu:257)
    CG_HD uint32_t open(Smem sm, const uint8_t *p, uint32_t len, uint32_t ring_col) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        wp = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        const uint32_t off = static_cast<uint32_t>(a & 3u) * 8u;
        end_bit = off + len * 8u;
        ring = ring_col;
        for (uint32_t j = 0; j < static_cast<uint32_t>(kRingRows); ++j) sm.st(ring + j * kTableRowBytes, fetch(j));
        loaded = kRingWords;
        // a stream that fits the ring never needs a top-up unless a (corrupt) stream is read far past its end
        next_refill = (end_bit <= static_cast<uint32_t>(kRingRows) * 32u) ? kRingWords * 32u : (kRingWords / 2) * 32u;
        pos = off;
        const uint32_t value = peek(sm);
        pos += 32u;
        return value;
    }
    CG_HD void refill(Smem sm) {
        do {
            for (uint32_t r = 0; r < static_cast<uint32_t>(kRingWords / 2); ++r) {
                const uint32_t j = loaded + r, row = j & static_cast<uint32_t>(kRingWords - 1);
                const uint32_t w = fetch(j);
                sm.st(ring + row * kTableRowBytes, w);
                if (row == 0u) sm.st(ring + kRingWords * kTableRowBytes, w);
            }
            loaded += kRingWords / 2;
        } while (loaded < (pos >> 5) + kRingWords / 2 + 1);
        next_refill = (loaded - kRingWords / 2) * 32u;
    }
    CG_HD void advance(Smem sm, uint32_t s) {
        pos += s;
        if (pos >= next_refill) refill(sm);
    }
};

// ---- decode loop ------------------------------------------------------------------------------------------
#ifndef CG_DEC_VARIANT
#define CG_DEC_VARIANT 2
#endif

CG_HD uint32_t cg_umulhi(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __umulhi(a, b);
#else
    return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}

// One step of the fast search: the candidate entry is IMM bytes above `a`; it is taken when
// hi32(spanm1 * c16) <= target.  That product is the exact (span * c16) >> 32 or one below it (it
// drops the "+ c16" of scale_by_cdf), so the search can end one entry too high when `target` sits
// exactly on a boundary; decode_symbol() checks the exact value afterwards.
template <uint32_t IMM>
CG_HD uint32_t search_step_fast(Smem sm, uint32_t a, uint32_t spanm1, uint32_t target) {
#if defined(__CUDA_ARCH__) && (CG_DEC_VARIANT & 1)
    asm("{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 c, h;\n\t"
        "ld.shared.u32 c, [%0+%3];\n\t"
        "mul.hi.u32 h, %1, c;\n\t"
        "setp.le.u32 p, h, %2;\n\t"
        "@p add.u32 %0, %0, %3;\n\t"
        "}"
        : "+r"(a)
        : "r"(spanm1), "r"(target), "n"(IMM));
    (void)sm;
    return a;
#else
    const uint32_t ca = a + IMM;
    return cg_umulhi(spanm1, sm.ld(ca)) <= target ? ca : a;
#endif
}

template <int B>
struct FastSearch {
    static CG_HD uint32_t run(Smem sm, uint32_t a, uint32_t spanm1, uint32_t target) {
        a = search_step_fast<(static_cast<uint32_t>(kTableRowBytes) << B)>(sm, a, spanm1, target);
        return FastSearch<B - 1>::run(sm, a, spanm1, target);
    }
};
template <>
struct FastSearch<-1> {
    static CG_HD uint32_t run(Smem, uint32_t a, uint32_t, uint32_t) { return a; }
};

// Exact search for tables whose symbol count is not a power of two: candidates above the last symbol
// are never taken (and never read).
template <int B>
struct ClampedSearch {
    static CG_HD uint32_t run(Smem sm, uint32_t a, uint32_t a_max, uint32_t spanm1, uint32_t target) {
        const uint32_t ca = a + (static_cast<uint32_t>(kTableRowBytes) << B);
        const bool ok = ca <= a_max;
        const bool take = ok && (scale_by_cdf(spanm1, sm.ld(ok ? ca : a)) <= target);
        return ClampedSearch<B - 1>::run(sm, take ? ca : a, a_max, spanm1, target);
    }
};
template <>
struct ClampedSearch<-1> {
    static CG_HD uint32_t run(Smem, uint32_t a, uint32_t, uint32_t, uint32_t) { return a; }
};

// Address of the table entry of the symbol under `target`, i.e. of the largest m in [0, maxsym] with
// (span * cdf[m]) >> 16 <= target (binsearch, dec_new.cu:52-71); *flo receives that scaled entry.
template <int LEVELS, bool POW2>
CG_HD uint32_t decode_symbol(Smem sm, uint32_t col, uint32_t a_max, uint32_t spanm1, uint32_t target,
                             uint32_t *flo) {
    uint32_t a;
    if (POW2) {
        a = FastSearch<LEVELS - 1>::run(sm, col, spanm1, target);
        *flo = scale_by_cdf(spanm1, sm.ld(a));
        if (*flo > target && a != col) {  // about once in 2^14 symbols
            a -= kTableRowBytes;
            *flo = scale_by_cdf(spanm1, sm.ld(a));
        }
    } else {
        a = ClampedSearch<LEVELS - 1>::run(sm, col, a_max, spanm1, target);
        *flo = scale_by_cdf(spanm1, sm.ld(a));
    }
    return a;
}

// col: address of the stream's table column; emit(i, a) receives the token index and the address of
// the decoded symbol's table entry (symbol = (a - col) / kTableRowBytes).
// LEVELS: search depth, 2^LEVELS >= maxsym + 1.  POW2: 2^LEVELS == maxsym + 1, so no candidate can
// exceed maxsym and the bound check is dropped.
//
// State: low, spanm1 = high - low, and offset = value - low.  In this form both kinds of
// renormalisation shift act alike on the pair (offset, span) -- offset = 2*offset + next bit,
// span = 2*span -- so the reference's "value -= 2^30" of the underflow case needs no separate step;
// low is still tracked because the shift counts depend on the bit patterns of low and high.
template <int LEVELS, bool POW2, class Emit>
CG_HD void decode_stream(Smem sm, uint32_t col, int maxsym, BitRing &bits, uint32_t value, int ntok, Emit emit) {
    uint32_t low = 0u, spanm1 = 0xFFFFFFFFu, offset = value;
    const uint32_t a_max = col + static_cast<uint32_t>(maxsym) * kTableRowBytes;
    for (int i = 0; i < ntok - 1; ++i) {
        const uint32_t win = bits.peek(sm);  // independent of this symbol's search: issued early
        uint32_t flo;
        const uint32_t a = decode_symbol<LEVELS, POW2>(sm, col, a_max, spanm1, offset, &flo);
        emit(i, a);
        const uint32_t fhi = (a == a_max) ? spanm1 + 1u : scale_by_cdf(spanm1, sm.ld(a + kTableRowBytes));
        offset -= flo;
        low += flo;
        spanm1 = fhi - flo - 1u;
        const uint32_t high = low + spanm1;
        // equal-top-bit shifts, then underflow shifts (dec_new.cu:283-301), applied in one go
        const uint32_t n1 = static_cast<uint32_t>(equal_shifts(low, high));
        const uint32_t k = static_cast<uint32_t>(cg_clz(((((~low) | high) << n1) << 1) | 1u));
        const uint32_t s = (n1 + k) & 31u;  // at most 18 for any strictly increasing table
        low = (low << s) & 0x7FFFFFFFu;
        spanm1 = cg_fshl(0xFFFFFFFFu, spanm1, s);
        offset = cg_fshl(win, offset, s);
        bits.advance(sm, s);
    }
    // the last symbol: no range update after it (dec_new.cu:273-275)
    uint32_t flo;
    emit(ntok - 1, decode_symbol<LEVELS, POW2>(sm, col, a_max, spanm1, offset, &flo));
}

// ---- MSB-first bit writer into one scratch row (add_bits_to_output, enc_new.cu:21-97) ---------------------
struct BitSink {
    uint32_t *row;    // 4-byte aligned scratch row of this stream
    uint32_t cap_w;   // words that fit in the row
    uint32_t nwords;  // words produced so far (may exceed cap_w: then nothing more is stored)
    uint64_t acc;     // pending output bits, right-aligned
    int nacc;         // number of bits in acc, < 32 between calls

    CG_HD void init(uint8_t *p, int64_t stride) {
        row = reinterpret_cast<uint32_t *>(p);
        cap_w = static_cast<uint32_t>(stride >> 2);
        nwords = 0;
        acc = 0;
        nacc = 0;
    }
    // appends the low n (0..32) bits of v (v has no bits above n)
    CG_HD void put(uint32_t v, int n) {
        acc = (acc << n) | v;
        nacc += n;
        if (nacc >= 32) {
            nacc -= 32;
            const uint32_t w = static_cast<uint32_t>(acc >> nacc);
            if (nwords < cap_w) row[nwords] = cg_bswap32(w);
            nwords++;
        }
    }
    // `count` copies of `bit`
    CG_HD void put_run(uint32_t bit, uint32_t count) {
        const uint32_t ones = 0u - bit;  // 0 or 0xFFFFFFFF
        while (count >= 32u) {
            put(ones, 32);
            count -= 32u;
        }
        if (count) put(ones >> (32u - count), static_cast<int>(count));
    }
    // zero-fills to a byte boundary; returns the stream length in bytes
    CG_HD uint32_t finish() {
        const uint32_t bytes = nwords * 4u + static_cast<uint32_t>((nacc + 7) >> 3);
        if (nacc) {
            const uint32_t w = static_cast<uint32_t>(acc << (32 - nacc));
            if (nwords < cap_w) row[nwords] = cg_bswap32(w);
        }
        return bytes;
    }
};

// ---- encoder state and step -----------------------------------------------------------------------------
struct EncoderState {
    uint32_t low, high, pending;
    CG_HD void init() {
        low = 0u;
        high = 0xFFFFFFFFu;
        pending = 0u;
    }
    // one symbol s in [0, maxsym] (enc_new.cu:257-295)
    CG_HD void step(Smem sm, uint32_t col, uint32_t s, uint32_t maxsym, BitSink &out) {
        const uint32_t a = col + s * kTableRowBytes;
        const uint32_t spanm1 = high - low;
        const uint32_t flo = scale_by_cdf(spanm1, sm.ld(a));
        const uint32_t fhi = (s == maxsym) ? spanm1 + 1u : scale_by_cdf(spanm1, sm.ld(a + kTableRowBytes));
        high = low + fhi - 1u;
        low = low + flo;
        // equal-top-bit shifts: their n1 bits are low's top bits; the first is followed by the pending
        // (inverted) bits of earlier underflow shifts (enc_new.cu:275-287)
        const int n1 = equal_shifts(low, high);
        if (n1) {
            const uint32_t bits = low >> (32 - n1);
            if (pending == 0u) {
                out.put(bits, n1);
            } else {
                const uint32_t first = bits >> (n1 - 1);
                out.put(first, 1);
                out.put_run(1u - first, pending);
                out.put(bits & ((1u << (n1 - 1)) - 1u), n1 - 1);
                pending = 0u;
            }
            low <<= n1;
            high = cg_fshl(0xFFFFFFFFu, high, static_cast<uint32_t>(n1));
        }
        // underflow shifts (enc_new.cu:288-293)
        const int k = underflow_shifts(low, high);
        pending += static_cast<uint32_t>(k);
        low = (low << k) & 0x7FFFFFFFu;
        high = cg_fshl(0xFFFFFFFFu, high, static_cast<uint32_t>(k)) | 0x80000000u;
    }
    // final flush (enc_new.cu:298-306); returns the stream length in bytes
    CG_HD uint32_t flush(BitSink &out) {
        pending += 1u;
        const uint32_t last = (low < 0x40000000u) ? 0u : 1u;
        out.put(last, 1);
        out.put_run(1u - last, pending);
        return out.finish();
    }
};

}  // namespace cg
