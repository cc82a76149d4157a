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

// Count of equal-top-bit shifts for the interval [low, high] (the |1 keeps it below 32 on a
// degenerate interval, which only a corrupt table can produce).
CG_HD int equal_shifts(uint32_t low, uint32_t high) { return cg_clz((low ^ high) | 1u); }
// ---- shared-memory access --------------------------------------------------------------------------------
// A stream's table is the column tab[m][tid] = cdf[m] << 16 of a [rows][128] uint32 array, addressed
// by byte address: entry m of the column starting at `col` is at col + m * kTableRowBytes.  On the
// device the addresses are shared-memory addresses (bank = lane for every row); on the host they are
// offsets into a plain array.
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

// ---- register bit window + warp-synchronous refill -----------------------------------------------------------
// The next 96 unread bits of the stream live in three registers.  The byte array is read as aligned
// 32-bit words; bits before the stream's first byte are shifted out at start-up and words (or word
// tails) past its last byte read as zero, which is what the reference sees in its zero-padded staging
// row (dec_new.cu:229-232).  A refill is taken by the whole warp as soon as any of its lanes is down to
// 32 bits and tops every lane up past 64 bits, so the refill code runs once per warp every few
// symbols instead of once per lane.
CG_HD bool cg_any_lane(uint32_t lanes, bool pred) {
#if defined(__CUDA_ARCH__)
    return __any_sync(lanes, pred) != 0;
#else
    (void)lanes;
    return pred;
#endif
}

CG_HD uint32_t cg_umulhi(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __umulhi(a, b);
#else
    return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}

struct BitWindow {
    const uint32_t *wp;    // word holding the stream's first byte
    uint32_t end_bit;      // bit index, counted from wp, one past the stream's last bit
    uint32_t next;         // next word to fetch
    uint32_t hi, mid, lo;  // unread bits, hi's top bit first
    int nbits;             // valid bits in hi:mid:lo

    CG_HD uint32_t fetch(uint32_t j) const {
        const uint32_t b0 = j * 32u;
        if (b0 >= end_bit) return 0u;
        uint32_t w = cg_bswap32(cg_load_stream_word(wp + j));
        const uint32_t rem = end_bit - b0;
        if (rem < 32u) w &= 0xFFFFFFFFu << (32u - rem);
        return w;
    }
    // returns the stream's first 32 bits (the coder's initial `value`, dec_new.cu:257)
    CG_HD uint32_t open(const uint8_t *p, uint32_t len) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        wp = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        const uint32_t off = static_cast<uint32_t>(a & 3u) * 8u;
        end_bit = off + len * 8u;
        const uint32_t w0 = fetch(0), w1 = fetch(1), w2 = fetch(2), w3 = fetch(3);
        hi = cg_fshl(w2, w1, off);
        mid = cg_fshl(w3, w2, off);
        lo = w3 << off;
        nbits = 96 - static_cast<int>(off);
        next = 4;
        return cg_fshl(w1, w0, off);
    }
    // drops the s (< 32) bits just shifted into the coder's value
    CG_HD void consume(uint32_t s) {
        hi = cg_fshl(mid, hi, s);
        mid = cg_fshl(lo, mid, s);
        lo <<= s;
        nbits -= static_cast<int>(s);
    }
    CG_HD bool low_water() const { return nbits <= 32; }
    CG_HD void refill() {
        while (nbits <= 64) {
            const uint32_t w = fetch(next++);
            const uint32_t p = static_cast<uint32_t>(nbits < 0 ? 0 : nbits);  // nothing valid below position p
            if (p < 32u) {
                hi |= cg_fshr_clamp(w, 0u, p);
                mid |= cg_fshl_clamp(0u, w, 32u - p);
            } else {
                mid |= cg_fshr_clamp(w, 0u, p - 32u);
                lo |= cg_fshl_clamp(0u, w, 64u - p);
            }
            nbits = static_cast<int>(p) + 32;
        }
    }
};

// ---- decode loop ------------------------------------------------------------------------------------------
// Scaled table entry for the current span: (span * c16) >> 32 with span32 = span mod 2^32, which is 0
// exactly when the range is the full 2^32 (then the product is c16 itself).
CG_HD uint32_t scale_exact(uint32_t span32, uint32_t c16) { return span32 ? cg_umulhi(span32, c16) : c16; }

// Search steps of the fast path (span32 != 0): the candidate entry is IMM bytes above `a`.
template <int B>
struct FastSearch {
    static CG_HD uint32_t run(Smem sm, uint32_t a, uint32_t span32, uint32_t target) {
        const uint32_t ca = a + (static_cast<uint32_t>(kTableRowBytes) << B);
        a = cg_umulhi(span32, sm.ld(ca)) <= target ? ca : a;
        return FastSearch<B - 1>::run(sm, a, span32, target);
    }
};
template <>
struct FastSearch<-1> {
    static CG_HD uint32_t run(Smem, uint32_t a, uint32_t, uint32_t) { return a; }
};

// Exact, clamped search: any table length, any span; candidates above the last symbol are never taken
// (and never read).
template <int B>
struct ExactSearch {
    static CG_HD uint32_t run(Smem sm, uint32_t a, uint32_t a_max, uint32_t span32, uint32_t target) {
        const uint32_t ca = a + (static_cast<uint32_t>(kTableRowBytes) << B);
        const bool ok = ca <= a_max;
        const bool take = ok && (scale_exact(span32, sm.ld(ok ? ca : a)) <= target);
        return ExactSearch<B - 1>::run(sm, take ? ca : a, a_max, span32, target);
    }
};
template <>
struct ExactSearch<-1> {
    static CG_HD uint32_t run(Smem, uint32_t a, uint32_t, uint32_t, uint32_t) { return a; }
};

// The decoder's arithmetic state: low, span32 = (high - low + 1) mod 2^32 and offset = value - low.
// In this form both kinds of renormalisation shift act alike on the pair (offset, span) --
// offset = 2*offset + next bit, span = 2*span -- so the reference's "value -= 2^30" of the underflow
// case needs no separate step; low is still tracked because the shift counts depend on the bit
// patterns of low and high.
struct DecoderState {
    uint32_t low, span32, offset;

    // range update for the symbol whose scaled bounds are [flo, fhi), then renormalisation
    // (dec_new.cu:277-301): equal-top-bit shifts and underflow shifts applied in one go
    CG_HD void update(uint32_t flo, uint32_t fhi, BitWindow &bw) {
        offset -= flo;
        low += flo;
        span32 = fhi - flo;
        const uint32_t high = low + span32 - 1u;
        const uint32_t n1 = static_cast<uint32_t>(equal_shifts(low, high));
        const uint32_t k = static_cast<uint32_t>(cg_clz(((((~low) | high) << n1) << 1) | 1u));
        const uint32_t s = n1 + k;  // at most 18 for any strictly increasing table; shifts below wrap at 32
        // The reference also clears low's top bit after underflow shifts.  Here low is only ever
        // compared with high = low + span - 1 bit by bit, offset carries value - low separately, and
        // a set top bit flips the top bit of low and high alike: it changes neither shift count.
        low = cg_fshl(0u, low, s);
        span32 = cg_fshl(0u, span32, s);
        offset = cg_fshl(bw.hi, offset, s);
        bw.consume(s);
    }
};

// One stream.  col: address of the stream's table column, entries cdf << 16, rows kTableRowBytes apart,
// one readable row past the last symbol's; emit(a) receives, token after token, the address of the
// decoded symbol's table entry (symbol = (a - col) / kTableRowBytes).  lanes: the warp's lanes that
// run this loop together (they must all have the same ntok).
// LEVELS: search depth, 2^LEVELS >= maxsym + 1.  POW2: 2^LEVELS == maxsym + 1 (with LEVELS >= 3): the
// middle symbols then take the fast path -- entries of the first two search levels in registers,
// no bound checks, one multiply-high per step -- and leave it only for a symbol that starts from the
// full 2^32 range (the first one, and about never again), which the exact path decodes.
template <int LEVELS, bool POW2, class Emit>
CG_HD void decode_stream(Smem sm, uint32_t col, int maxsym, const uint8_t *stream, uint32_t len, int ntok,
                         uint32_t lanes, Emit emit) {
    BitWindow bw;
    DecoderState st;
    st.low = 0u;
    st.span32 = 0u;
    st.offset = bw.open(stream, len);
    const uint32_t a_max = col + static_cast<uint32_t>(maxsym) * kTableRowBytes;

    // exact step; with_update = false for the last symbol (dec_new.cu:273-275)
    auto exact_step = [&](bool with_update) {
        const uint32_t a = ExactSearch<LEVELS - 1>::run(sm, col, a_max, st.span32, st.offset);
        emit(a);
        if (with_update) {
            const uint32_t flo = scale_exact(st.span32, sm.ld(a));
            const uint32_t fhi = (a == a_max) ? st.span32 : scale_exact(st.span32, sm.ld(a + kTableRowBytes));
            st.update(flo, fhi, bw);
        }
    };

    constexpr bool kFast = POW2 && LEVELS >= 3;
    constexpr uint32_t kTop = static_cast<uint32_t>(kTableRowBytes) << (LEVELS > 0 ? LEVELS - 1 : 0);
    constexpr uint32_t kHalf = kTop >> 1;
    uint32_t r_mid = 0u, r_lo = 0u, r_hi = 0u;
    if (kFast) {
        r_mid = sm.ld(col + kTop);
        r_lo = sm.ld(col + kHalf);
        r_hi = sm.ld(col + kTop + kHalf);
    }
    for (int left = ntok - 1; left > 0; --left) {
        // rare, and taken by the whole warp: a lane is low on bits, or starts this symbol from the full range
        if (cg_any_lane(lanes, bw.low_water() || (kFast && st.span32 == 0u)) || !kFast) {
            if (cg_any_lane(lanes, bw.low_water())) bw.refill();
            if (!kFast || cg_any_lane(lanes, st.span32 == 0u)) {
                exact_step(true);
                continue;
            }
        }
        // levels 1 and 2 from registers, the rest from the table column
        const bool t1 = cg_umulhi(st.span32, r_mid) <= st.offset;
        uint32_t a = t1 ? col + kTop : col;
        const bool t2 = cg_umulhi(st.span32, t1 ? r_hi : r_lo) <= st.offset;
        a = t2 ? a + kHalf : a;
        a = FastSearch<(kFast ? LEVELS - 3 : -1)>::run(sm, a, st.span32, st.offset);
        emit(a);
        const uint32_t flo = cg_umulhi(st.span32, sm.ld(a));
        const uint32_t fnext = cg_umulhi(st.span32, sm.ld(a + kTableRowBytes));
        st.update(flo, (a == a_max) ? st.span32 : fnext, bw);
    }
    if (cg_any_lane(lanes, bw.low_water())) bw.refill();
    exact_step(false);
}

// ---- MSB-first bit writer into one scratch row (add_bits_to_output, enc_new.cu:21-97) ---------------------
// Output bits collect in a 64-bit accumulator.  Whole 32-bit words leave it, big-endian, into the
// stream's scratch row; the common case does that for the whole warp at once (see EncoderState::step)
// so that the store is not a per-lane branch.
struct BitSink {
    uint32_t *row;    // 4-byte aligned scratch row of this stream
    uint32_t cap_w;   // words that fit in the row
    uint32_t nwords;  // words produced so far (may exceed cap_w: then nothing more is stored)
    uint64_t acc;     // pending output bits, right-aligned
    uint32_t nacc;    // number of bits in acc, < 64

    CG_HD void init(uint8_t *p, int64_t stride) {
        row = reinterpret_cast<uint32_t *>(p);
        cap_w = static_cast<uint32_t>(stride >> 2);
        nwords = 0;
        acc = 0;
        nacc = 0;
    }
    // appends the low n bits of v (v has no bits above n); needs nacc + n <= 64
    CG_HD void put(uint32_t v, uint32_t n) {
        acc = (acc << n) | v;
        nacc += n;
    }
    // moves the oldest 32 bits out; needs nacc >= 32
    CG_HD void store_word() {
        nacc -= 32u;
        const uint32_t w = static_cast<uint32_t>(acc >> nacc);
        if (nwords < cap_w) row[nwords] = cg_bswap32(w);
        nwords++;
    }
    CG_HD void drain() {
        while (nacc >= 32u) store_word();
    }
    // `count` copies of `bit`, any count
    CG_HD void put_run(uint32_t bit, uint32_t count) {
        const uint32_t ones = 0u - bit;  // 0 or 0xFFFFFFFF
        while (count) {
            drain();
            const uint32_t n = count < 32u ? count : 32u;
            put(ones >> (32u - n), n);
            count -= n;
        }
    }
    // zero-fills to a byte boundary; returns the stream length in bytes
    CG_HD uint32_t finish() {
        drain();
        const uint32_t bytes = nwords * 4u + ((nacc + 7u) >> 3);
        if (nacc) {
            const uint32_t w = static_cast<uint32_t>(acc << (32u - nacc));
            if (nwords < cap_w) row[nwords] = cg_bswap32(w);
        }
        return bytes;
    }
};

// ---- encoder state and step -----------------------------------------------------------------------------
constexpr uint32_t kSinkHighWater = 48;  // a symbol starts with fewer bits than this in the accumulator
constexpr uint32_t kFastEmitBits = 16;   // ... so up to this many more fit without a store

struct EncoderState {
    uint32_t low, span32, pending;  // span32 = (high - low + 1) mod 2^32, 0 for the full range
    CG_HD void init() {
        low = 0u;
        span32 = 0u;
        pending = 0u;
    }
    // one symbol s in [0, maxsym] (enc_new.cu:257-295); the table column must have a readable row
    // after the last symbol's.  lanes: the warp's lanes that encode together (same token count).
    CG_HD void step(Smem sm, uint32_t col, uint32_t s, uint32_t maxsym, BitSink &out, uint32_t lanes) {
        const uint32_t a = col + s * kTableRowBytes;
        const uint32_t flo = scale_exact(span32, sm.ld(a));
        const uint32_t fnext = scale_exact(span32, sm.ld(a + kTableRowBytes));
        const uint32_t fhi = (s == maxsym) ? span32 : fnext;
        low += flo;
        span32 = fhi - flo;
        const uint32_t high = low + span32 - 1u;
        // equal-top-bit shifts: their n1 bits are low's top bits; the first is followed by the pending
        // (inverted) bits of earlier underflow shifts (enc_new.cu:275-287)
        const uint32_t n1 = static_cast<uint32_t>(equal_shifts(low, high));
        if (n1) {
            const uint32_t bits = low >> (32u - n1);
            const uint32_t first = bits >> (n1 - 1u);
            const uint32_t rest = bits & ((1u << (n1 - 1u)) - 1u);
            const uint32_t total = n1 + pending;
            if (total <= kFastEmitBits) {
                const uint32_t run = ((1u << pending) - 1u) & (first - 1u);  // pending ones after a 0, zeros after a 1
                out.put((first << (total - 1u)) | (run << (n1 - 1u)) | rest, total);
            } else {
                out.drain();
                out.put(first, 1u);
                out.put_run(1u - first, pending);
                out.drain();
                out.put(rest, n1 - 1u);
            }
            pending = 0u;
        }
        // underflow shifts (enc_new.cu:288-293) only raise the pending count; both kinds of shift
        // double the span
        const uint32_t k = static_cast<uint32_t>(cg_clz(((((~low) | high) << n1) << 1) | 1u));
        pending += k;
        const uint32_t sh = (n1 + k) & 31u;
        low = (low << sh) & 0x7FFFFFFFu;
        span32 <<= sh;
        // a store for every lane that has a full word, as soon as one lane is near the high-water mark
        if (cg_any_lane(lanes, out.nacc >= kSinkHighWater)) {
            if (out.nacc >= 32u) out.store_word();
        }
    }
    // final flush (enc_new.cu:298-306); returns the stream length in bytes
    CG_HD uint32_t flush(BitSink &out) {
        pending += 1u;
        const uint32_t last = (low < 0x40000000u) ? 0u : 1u;
        out.drain();
        out.put(last, 1u);
        out.put_run(1u - last, pending);
        return out.finish();
    }
};

}  // namespace cg
