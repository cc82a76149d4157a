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
    for (int m = 0; m < lp; ++m) tab[m * kGroupChannels + tid] = static_cast<uint32_t>(cdf[m]) << 16;
    for (int m = lp; m < rows; ++m) tab[m * kGroupChannels + tid] = 0u;
    return tab;
}

extern "C" int64_t hm_encode_stream(const uint16_t *cdf, int lp, const int8_t *sym, int n, uint8_t *out,
                                    int64_t cap, int tid) {
    std::vector<uint32_t> tab = make_table(cdf, lp, lp, tid);
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
    std::vector<uint32_t> tab = make_table(cdf, lp - 1 < rows ? lp - 1 : rows, rows, tid);
    tab.resize(static_cast<size_t>(rows + 1) * kGroupChannels, 0xDEADBEEFu);
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

