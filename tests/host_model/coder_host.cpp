// Host build of the product's per-stream coder loops (cachegen_b200/csrc/cg_coder.cuh), for the CPU
// test-suite only: lets the tests drive the exact decode/encode step code against the oracle without
// a GPU.  Not part of the shipped library.
#include <cstring>
#include <vector>

#include "../../cachegen_b200/csrc/cg_coder.cuh"

using namespace cg;

static int search_levels(int lp) {
    int n = 0;
    while ((1 << n) < lp - 1) n++;
    return n;
}

// The table column of lane `tid` inside a [rows][128] uint32 array, as the kernels stage it.
static std::vector<uint32_t> make_table(const uint16_t *cdf, int lp, int rows, int tid) {
    std::vector<uint32_t> tab(static_cast<size_t>(rows) * kGroupChannels, 0xDEADBEEFu);
    for (int m = 0; m < lp && m < rows; ++m) tab[m * kGroupChannels + tid] = static_cast<uint32_t>(cdf[m]) << 16;
    for (int m = lp; m < rows; ++m) tab[m * kGroupChannels + tid] = 0xFFFFFFFFu;  // the kernels' padding
    return tab;
}

extern "C" int64_t hm_encode_stream(const uint16_t *cdf, int lp, const int8_t *sym, int n, uint8_t *out,
                                    int64_t cap, int tid) {
    std::vector<uint32_t> tab = make_table(cdf, lp - 1, lp, tid);
    Smem rd{reinterpret_cast<uint8_t *>(tab.data())};
    const uint32_t col = static_cast<uint32_t>(tid) * 4u;
    BitSink sink;
    sink.init(out, cap);
    EncoderState enc;
    enc.init();
    for (int i = 0; i < n; ++i) enc.step(rd, col, static_cast<uint8_t>(sym[i]), static_cast<uint32_t>(lp - 2), sink, 0xFFFFFFFFu);
    return enc.flush(sink);
}

template <int LEVELS, bool POW2>
static void run_decode(const uint16_t *cdf, int lp, const uint8_t *bytes, int64_t len, int n, uint8_t *out,
                              int tid) {
    const int rows = (1 << LEVELS) > lp - 1 ? (1 << LEVELS) : lp - 1;
    std::vector<uint32_t> tab = make_table(cdf, lp - 1 < rows ? lp - 1 : rows, rows + 1, tid);
    Smem rd{reinterpret_cast<uint8_t *>(tab.data())};
    decode_stream<LEVELS, POW2>(rd, static_cast<uint32_t>(tid) * 4u, lp - 2, bytes, static_cast<uint32_t>(len),
                                       n, 0xFFFFFFFFu, [&](uint32_t a) {
                                           *out++ = static_cast<uint8_t>((a - static_cast<uint32_t>(tid) * 4u) /
                                                                         kTableRowBytes);
                                       });
}

extern "C" void hm_decode_stream(const uint16_t *cdf, int lp, const uint8_t *bytes, int64_t len, int n,
                                        uint8_t *out, int tid) {
    const int need = search_levels(lp);
    const bool pow2 = (1 << need) == lp - 1;
    if (pow2 && need == 5) run_decode<5, true>(cdf, lp, bytes, len, n, out, tid);
    else if (pow2 && need == 4) run_decode<4, true>(cdf, lp, bytes, len, n, out, tid);
    else if (pow2 && need == 3) run_decode<3, true>(cdf, lp, bytes, len, n, out, tid);
    else if (need <= 3) run_decode<3, false>(cdf, lp, bytes, len, n, out, tid);
    else if (need == 4) run_decode<4, false>(cdf, lp, bytes, len, n, out, tid);
    else if (need == 5) run_decode<5, false>(cdf, lp, bytes, len, n, out, tid);
    else run_decode<6, false>(cdf, lp, bytes, len, n, out, tid);
}


// Two streams side by side through decode_streams, as the two-channels-per-thread kernel runs them:
// tables in columns tid and tid + 64, search depth fl forced by the caller (any depth must give the
// same symbols).  out receives the symbols interleaved: out[2 * token + stream].
template <int FL>
static void run_pair(const uint16_t *cdf0, const uint16_t *cdf1, int lp, const uint8_t *b0, int64_t l0,
                     const uint8_t *b1, int64_t l1, int n, uint8_t *out, int tid) {
    const int full = search_levels(lp);
    const int lv = full < 2 ? 2 : full;
    const int rows = ((1 << lv) > lp - 1 ? (1 << lv) : lp - 1) + 1;
    std::vector<uint32_t> tab = make_table(cdf0, lp - 1, rows, tid);
    const std::vector<uint32_t> t1 = make_table(cdf1, lp - 1, rows, tid + 64);
    for (int m = 0; m < rows; ++m) tab[m * kGroupChannels + tid + 64] = t1[m * kGroupChannels + tid + 64];
    Smem rd{reinterpret_cast<uint8_t *>(tab.data())};
    const uint32_t col[2] = {static_cast<uint32_t>(tid) * 4u, static_cast<uint32_t>(tid + 64) * 4u};
    const int maxsym = lp - 2, top = (1 << FL) - 1;
    const uint32_t det = static_cast<uint32_t>(top < maxsym ? top : maxsym) * kTableRowBytes;
    const uint8_t *const streams[2] = {b0, b1};
    const uint32_t lens[2] = {static_cast<uint32_t>(l0), static_cast<uint32_t>(l1)};
    decode_streams<FL, 2>(rd, col, det, maxsym, full, streams, lens, n, 0xFFFFFFFFu, [&](const uint32_t(&a)[2], uint32_t) {
        *out++ = static_cast<uint8_t>((a[0] - col[0]) / kTableRowBytes);
        *out++ = static_cast<uint8_t>((a[1] - col[1]) / kTableRowBytes);
    });
}

extern "C" int hm_decode_pair(const uint16_t *cdf0, const uint16_t *cdf1, int lp, const uint8_t *b0, int64_t l0,
                              const uint8_t *b1, int64_t l1, int n, uint8_t *out, int tid, int fl) {
    const int full = search_levels(lp);
    if (fl < 2 || fl > 6 || (fl > full && fl > 2) || tid < 0 || tid >= 64) return -1;
    switch (fl) {
    case 2: run_pair<2>(cdf0, cdf1, lp, b0, l0, b1, l1, n, out, tid); break;
    case 3: run_pair<3>(cdf0, cdf1, lp, b0, l0, b1, l1, n, out, tid); break;
    case 4: run_pair<4>(cdf0, cdf1, lp, b0, l0, b1, l1, n, out, tid); break;
    case 5: run_pair<5>(cdf0, cdf1, lp, b0, l0, b1, l1, n, out, tid); break;
    default: run_pair<6>(cdf0, cdf1, lp, b0, l0, b1, l1, n, out, tid); break;
    }
    return 0;
}

extern "C" int hm_fast_levels_for(int nsym, int full_levels) { return fast_levels_for(nsym, full_levels); }
