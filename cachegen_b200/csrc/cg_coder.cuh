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
// x << n, 0 for n >= 32.  On the device a clamping funnel shift: a plain `<<` by 32 or more is undefined
// to the compiler, which may then emit the wrapping form.
CG_HD uint32_t cg_shl(uint32_t x, uint32_t n) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_lc(0u, x, n);
#else
    return n >= 32u ? 0u : x << n;
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

    // word j of the stream, big-endian, bits past the stream's end cleared; no branches
    CG_HD uint32_t fetch(uint32_t j) const {
        const uint32_t b0 = j * 32u;
        uint32_t w = 0u;
        if (b0 < end_bit) w = cg_bswap32(cg_load_stream_word(wp + j));
        const uint32_t rem = end_bit - b0;  // >= 2^31 (clamped to 32 below) when the word lies past the end
        return w & ~cg_fshr_clamp(0xFFFFFFFFu, 0u, rem);
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
    // fewer valid bits than one symbol can take: a range update shifts by at most 18 bits when the
    // table is strictly increasing (the updated interval spans at least 2^14 values)
    CG_HD bool short_of_bits() const { return nbits < 18; }
    // Tops the window up with the whole words that fit (none above 64 valid bits, one above 32, two
    // otherwise), straight-line: every lane of the warp runs the same instructions whatever it needs.
    CG_HD void refill() {
        const uint32_t p = static_cast<uint32_t>(nbits < 0 ? 0 : nbits);  // nothing valid below position p
        const uint32_t k = p <= 32u ? 2u : (p <= 64u ? 1u : 0u);
        uint32_t wa = fetch(next), wb = fetch(next + 1u);
        if (k < 2u) wb = 0u;
        if (k < 1u) wa = 0u;
        // (wa:wb) goes to bit position p of hi:mid:lo, whose bits from p on are zero
        const uint32_t q = p & 31u;
        const uint32_t t0 = cg_fshr_clamp(wa, 0u, q);        // wa >> q
        const uint32_t t1 = cg_fshr_clamp(wb, wa, q);        // low word of (wa:wb) >> q
        const uint32_t t2 = cg_fshl_clamp(0u, wb, 32u - q);  // wb << (32 - q), 0 for q == 0
        if (p < 32u) {
            hi |= t0;
            mid |= t1;
            lo |= t2;
        } else if (p < 64u) {  // one word fits past position 32, or two exactly at it (q == 0: t1 == wb)
            mid |= t0;
            lo |= t1;
        } else {  // a word fits only at position 64 exactly (wa is 0 beyond it)
            lo |= t0;
        }
        nbits = static_cast<int>(p + 32u * k);
        next += k;
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

// The same update for the decode_streams loop: no "| 1" guards on the two leading-zero counts.  With a
// strictly increasing table the updated interval spans at least 2^14 values, so neither operand can be
// zero; on a corrupt table a count of 32 only makes the shifts below wrap, and every later read stays
// inside the table column and the stream.
CG_HD void update_unguarded(DecoderState &st, uint32_t flo, uint32_t fhi, BitWindow &bw) {
    st.offset -= flo;
    st.low += flo;
    st.span32 = fhi - flo;
    const uint32_t high = st.low + st.span32 - 1u;
    const uint32_t n1 = static_cast<uint32_t>(cg_clz(st.low ^ high));
    const uint32_t y = cg_shl((~st.low) | high, n1);  // top bit set: low has 0 and high 1 at the first bit they differ in
    const uint32_t s = n1 + static_cast<uint32_t>(cg_clz(y + y));
    st.low = cg_fshl(0u, st.low, s);
    st.span32 = cg_fshl(0u, st.span32, s);
    st.offset = cg_fshl(bw.hi, st.offset, s);
    bw.consume(s);
}

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

// ---- decode loop, NS streams per lane, search depth chosen by the caller ---------------------------------
// Exact search with a run-time depth (the rare path of decode_streams).
CG_HD uint32_t exact_search(Smem sm, uint32_t col, uint32_t a_max, uint32_t span32, uint32_t target, int levels) {
    uint32_t a = col;
    for (int b = levels - 1; b >= 0; --b) {
        const uint32_t ca = a + (static_cast<uint32_t>(kTableRowBytes) << b);
        const bool ok = ca <= a_max;
        const bool take = ok && (scale_exact(span32, sm.ld(ok ? ca : a)) <= target);
        a = take ? ca : a;
    }
    return a;
}

// Smallest search depth whose top entry, 2^depth - 1, lies above every symbol 0 .. nsym-1, kept
// within [2, full_levels].
CG_HD int fast_levels_for(int nsym, int full_levels) {
    int fl = 2;
    while (fl < full_levels && (1 << fl) - 1 < nsym) fl++;
    return fl;
}

// NS streams of one lane decoded side by side (same token count, same table length), the fast
// search limited to the first 2^FL table entries.
//
// The caller picks FL from what it knows about the symbols (a row quantised to `bins` bins holds
// symbols 0 .. bins-2, so 2^FL >= bins is enough); the result never depends on that choice: a fast
// search that ends on or above entry D = min(2^FL - 1, maxsym) -- the only way a symbol >= D, a
// symbol that starts from the full 2^32 range (span32 == 0 makes every comparison true) or a probe
// of a padding entry can show -- is thrown away and the whole warp repeats that symbol with the
// exact, full-depth search.  Entries above maxsym must be staged as 0xFFFFFFFF (never "<= offset"
// unless offset is span-1, which then lands above D) and the column needs 2^FL + 1 readable rows.
//   col[i]    table column of stream i (see decode_stream)
//   det       address threshold of entry D: column-independent because a column's offset inside a
//             table row is below kTableRowBytes (det = table base + D * kTableRowBytes)
//   emit(a, t4)  receives the NS table-entry addresses of one token's symbols and four times the
//             token's index (ntok >= 1)
template <int FL, int NS, class Emit>
CG_HD void decode_streams(Smem sm, const uint32_t (&col)[NS], uint32_t det, int maxsym, int full_levels,
                          const uint8_t *const (&stream)[NS], const uint32_t (&len)[NS], int ntok, uint32_t lanes,
                          Emit emit) {
    static_assert(FL >= 2, "the first two levels are held in registers");
    BitWindow bw[NS];
    DecoderState st[NS];
    uint32_t r_mid[NS], r_lo[NS], r_hi[NS], a_max[NS], col_top[NS];
    constexpr uint32_t kTop = static_cast<uint32_t>(kTableRowBytes) << (FL - 1);
    constexpr uint32_t kHalf = kTop >> 1;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < NS; ++i) {
        st[i].low = 0u;
        st[i].span32 = 0u;
        st[i].offset = bw[i].open(stream[i], len[i]);
        a_max[i] = col[i] + static_cast<uint32_t>(maxsym) * kTableRowBytes;
        col_top[i] = col[i] + kTop;
        r_mid[i] = sm.ld(col[i] + kTop);
        r_lo[i] = sm.ld(col[i] + kHalf);
        r_hi[i] = sm.ld(col[i] + kTop + kHalf);
    }
    uint32_t a[NS];
    // One back edge and one vote per token: the rare path (a refill of the bit windows, or the exact
    // search when the fast one cannot be trusted) only tops the windows up or replaces the symbol and
    // its scaled bounds; the range update below is shared.
    const uint32_t last4 = static_cast<uint32_t>(ntok - 1) * 4u;
    uint32_t t4 = 0u;  // four times the token index: the caller's emit indexes 4-byte per-token data with it
    for (; t4 != last4; t4 += 4u) {
        uint32_t flo[NS], fhi[NS];
        bool rare = false;  // a lane short of bits, or a search that ended on or above entry D
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < NS; ++i) {
            const bool t1 = cg_umulhi(st[i].span32, r_mid[i]) <= st[i].offset;
            uint32_t x = t1 ? col_top[i] : col[i];
            a[i] = cg_umulhi(st[i].span32, t1 ? r_hi[i] : r_lo[i]) <= st[i].offset ? x + kHalf : x;
        }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < NS; ++i) a[i] = FastSearch<FL - 3>::run(sm, a[i], st[i].span32, st[i].offset);
        uint32_t e0[NS], e1[NS];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < NS; ++i) {
            e0[i] = sm.ld(a[i]);
            e1[i] = sm.ld(a[i] + kTableRowBytes);
        }
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < NS; ++i) {
            rare = rare || a[i] >= det || bw[i].short_of_bits();
            flo[i] = cg_umulhi(st[i].span32, e0[i]);
            fhi[i] = cg_umulhi(st[i].span32, e1[i]);
        }
        if (cg_any_lane(lanes, rare)) {
            bool low = false, odd = false;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
            for (int i = 0; i < NS; ++i) {
                low = low || bw[i].short_of_bits();
                odd = odd || a[i] >= det;
            }
            if (cg_any_lane(lanes, low)) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
                for (int i = 0; i < NS; ++i) bw[i].refill();
            }
            if (cg_any_lane(lanes, odd)) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
                for (int i = 0; i < NS; ++i) {
                    a[i] = exact_search(sm, col[i], a_max[i], st[i].span32, st[i].offset, full_levels);
                    flo[i] = scale_exact(st[i].span32, sm.ld(a[i]));
                    fhi[i] = (a[i] == a_max[i]) ? st[i].span32
                                                : scale_exact(st[i].span32, sm.ld(a[i] + kTableRowBytes));
                }
            }
        }
        emit(a, t4);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int i = 0; i < NS; ++i) update_unguarded(st[i], flo[i], fhi[i], bw[i]);
    }
    // last symbol: no range update (dec_new.cu:273-275), so no new bits either
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < NS; ++i) a[i] = exact_search(sm, col[i], a_max[i], st[i].span32, st[i].offset, full_levels);
    emit(a, t4);
}

// ---- MSB-first bit writer into one scratch row (add_bits_to_output, enc_new.cu:21-97) ---------------------
// Output bits collect in a 64-bit accumulator.  Whole 32-bit words leave it, big-endian, into the
// stream's scratch row; the common case does that for the whole warp at once (see EncoderState::step)
// so that the store is not a per-lane branch.
struct BitSink {
    uint32_t *row;    // 4-byte aligned scratch row of this stream
    uint32_t cap_w;   // words that fit in the row
    uint32_t nwords;  // words produced so far (may exceed cap_w: then nothing more is stored)
    uint32_t acc_hi, acc_lo;  // pending output bits, right-aligned in (acc_hi:acc_lo)
    uint32_t nacc;            // number of bits pending, < 64

    CG_HD void init(uint8_t *p, int64_t stride) {
        row = reinterpret_cast<uint32_t *>(p);
        cap_w = static_cast<uint32_t>(stride >> 2);
        nwords = 0;
        acc_hi = 0;
        acc_lo = 0;
        nacc = 0;
    }
    // appends the low n bits of v (v has no bits above n), n <= 32; needs nacc + n <= 64
    CG_HD void put(uint32_t v, uint32_t n) {
        acc_hi = cg_fshl_clamp(acc_lo, acc_hi, n);
        acc_lo = cg_shl(acc_lo, n) | v;
        nacc += n;
    }
    // the same for n < 32 (what the straight-line encoder step appends): plain funnel shifts
    CG_HD void put_short(uint32_t v, uint32_t n) {
        acc_hi = cg_fshl(acc_lo, acc_hi, n);
        acc_lo = acc_lo * cg_shl(1u, n) + v;  // a multiply-add for shift and or: off the integer pipe, which binds the encoder
        nacc += n;
    }
    // moves the oldest 32 bits out; needs nacc >= 32
    CG_HD void store_word() {
        nacc -= 32u;
        const uint32_t w = cg_fshr_clamp(acc_lo, acc_hi, nacc);  // nacc < 32: the low word of (hi:lo) >> nacc
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
            const uint32_t w = acc_lo << (32u - nacc);  // after drain: 0 < nacc < 32
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
    // 1 and -1 as values the compiler cannot see through (the kernel reads them from constant memory):
    // a + b written as a * one + b is a multiply-add, which keeps it off the integer pipe that binds the
    // encoder's step; a plain a + b would be folded back into an integer add
    uint32_t one, minus_one;
    CG_HD void init(uint32_t opaque_one = 1u, uint32_t opaque_minus_one = 0xFFFFFFFFu) {
        low = 0u;
        span32 = 0u;
        pending = 0u;
        one = opaque_one;
        minus_one = opaque_minus_one;
    }
    CG_HD uint32_t add_f(uint32_t a, uint32_t b) const { return a * one + b; }
    CG_HD uint32_t sub_f(uint32_t a, uint32_t b) const { return b * minus_one + a; }  // a - b
    // One symbol s in [0, maxsym] (enc_new.cu:257-295), any state, any number of output bits; stores
    // whole words as needed but leaves up to 63 bits in the accumulator.  The table column must have
    // a readable row after the last symbol's.
    CG_HD void step_general(Smem sm, uint32_t col, uint32_t s, uint32_t maxsym, BitSink &out) {
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
            out.drain();
            out.put(first, 1u);
            out.put_run(1u - first, pending);
            out.drain();
            out.put(rest, n1 - 1u);
            pending = 0u;
        }
        // underflow shifts (enc_new.cu:288-293) only raise the pending count; both kinds of shift
        // double the span
        const uint32_t k = static_cast<uint32_t>(cg_clz(((((~low) | high) << n1) << 1) | 1u));
        pending += k;
        const uint32_t sh = (n1 + k) & 31u;
        low = (low << sh) & 0x7FFFFFFFu;
        span32 <<= sh;
    }
    // The same symbol in straight-line code for the usual case -- the range is not the full 2^32 (it is
    // only for a stream's first symbol, and after a shift that lands on it exactly) and at most
    // kFastEmitBits bits come out.  step_try does the step on that assumption and says whether it held
    // (`before` keeps what is needed to take the step again); step_finish repairs a lane for which
    // it did not, through step_general, and stores a full word of the accumulator.  Between the two
    // goes ONE warp vote (see step), so that neither the repair nor the store is a per-lane branch in
    // the usual case.
    struct Before {
        uint32_t low, span32, pending, nacc, acc_hi, acc_lo;
    };
    CG_HD bool step_try(Smem sm, uint32_t col, uint32_t s, uint32_t maxsym, BitSink &out, Before &before) {
        before.low = low;
        before.span32 = span32;
        before.pending = pending;
        before.nacc = out.nacc;
        before.acc_hi = out.acc_hi;
        before.acc_lo = out.acc_lo;
        const uint32_t a = col + s * kTableRowBytes;
        const uint32_t flo = cg_umulhi(span32, sm.ld(a));
        const uint32_t fnext = cg_umulhi(span32, sm.ld(a + kTableRowBytes));
        const uint32_t fhi = (s == maxsym) ? span32 : fnext;
        low = add_f(low, flo);
        span32 = sub_f(fhi, flo);
        const uint32_t high = low + span32 - 1u;
        // low == high (32 here) and k == 32 below only come from a table that is not increasing: the first
        // sends the lane to the general path (total > kFastEmitBits), the second makes the shifts give 0
        const uint32_t n1 = static_cast<uint32_t>(cg_clz(low ^ high));
        const uint32_t y = cg_shl((~low) | high, n1);
        const uint32_t k = static_cast<uint32_t>(cg_clz(y + y));
        // Output when n1 != 0: low's top bit, then the pending bits as its inverse, then low's next
        // n1 - 1 bits.  As a number that is (2^q - 1) * 2^(n1 - 1) + (low's top n1 bits), q the pending
        // count: the sum carries into the top bit's place exactly when that bit is 1.  With n1 == 0 nothing
        // goes out: q is taken as 0 then, which makes the value 0 and the bit count 0 without a mask.  A
        // lane that has to take the step again may append anything: step_finish puts its accumulator back.
        const uint32_t q = n1 ? pending : 0u;
        const uint32_t nput = add_f(n1, q);
        const bool redo = (before.span32 == 0u) | (nput > kFastEmitBits);
        const uint32_t ones = cg_shl(1u, q) - 1u;
        out.put_short(cg_shl(ones, n1 - 1u) + cg_fshl(low, 0u, n1), nput);
        pending = add_f(sub_f(pending, q), k);
        const uint32_t sh = add_f(n1, k);  // at most 18 with an increasing table
        const uint32_t p2 = cg_shl(1u, sh);  // one shift and two multiplies for two shifts: see put_short
        low = (low * p2) & 0x7FFFFFFFu;
        span32 = span32 * p2;
        return redo;
    }
    CG_HD void step_finish(bool redo, const Before &before, Smem sm, uint32_t col, uint32_t s, uint32_t maxsym,
                           BitSink &out) {
        if (redo) {
            low = before.low;
            span32 = before.span32;
            pending = before.pending;
            out.acc_hi = before.acc_hi;
            out.acc_lo = before.acc_lo;
            out.nacc = before.nacc;
            step_general(sm, col, s, maxsym, out);
        }
        if (out.nacc >= 32u) out.store_word();
    }
    // One symbol of one stream per lane.  lanes: the warp's lanes that encode together (same token
    // count).  Every lane with a full word stores it as soon as one lane is near the accumulator's
    // high-water mark.
    CG_HD void step(Smem sm, uint32_t col, uint32_t s, uint32_t maxsym, BitSink &out, uint32_t lanes) {
        Before before;
        const bool redo = step_try(sm, col, s, maxsym, out, before);
        if (cg_any_lane(lanes, redo || out.nacc >= kSinkHighWater)) step_finish(redo, before, sm, col, s, maxsym, out);
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
