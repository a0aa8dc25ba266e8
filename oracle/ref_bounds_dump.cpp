// TEST INFRASTRUCTURE.  Compiled against the reference's cuda/common.cuh where it
// lies (include path given on the command line, nothing is copied) to dump the
// outputs of its host-callable helpers sg_row_bounds, sg_col_bounds and
// sg_pack_mask32 as JSON.  tests/golden/make_golden.py runs it and commits the
// output as tests/golden/bounds.json, which pins att3_sg_tile_ranges and
// att3_pack_mask32.
#include "common.cuh"

#include <cstdio>
#include <random>
#include <vector>

int main() {
    const int cases[][2] = {{1, 1}, {15, 7}, {16, 0}, {16, 1}, {17, 16}, {31, 32}, {32, 32}, {33, 7}, {33, 33},
                            {48, 48}, {63, 31}, {64, 0}, {64, 7}, {64, 16}, {65, 32}, {80, 33}, {96, 32}, {96, 40},
                            {127, 32}, {128, 0}, {128, 128}, {129, 1}, {129, 136}, {256, 32}, {257, 32}, {272, 40}};
    const int tiles[][2] = {{32, 16}, {32, 32}, {64, 32}, {128, 64}};
    std::printf("{\"ranges\": [");
    bool first = true;
    for (auto& c : cases)
        for (auto& t : tiles)
            for (int side = 0; side < 2; ++side)
                for (int a = 0; a < c[0]; a += (c[0] > 64 ? 7 : 1)) {
                    int lo, hi;
                    sg_row_bounds(side, a, c[0], c[1], t[0], lo, hi);
                    std::printf("%s{\"N\":%d,\"w\":%d,\"bj\":%d,\"bk\":%d,\"side\":%d,\"a\":%d,\"blocks\":[",
                                first ? "" : ",", c[0], c[1], t[0], t[1], side, a);
                    first = false;
                    bool f2 = true;
                    for (int j0 = lo; j0 < hi; j0 += t[0]) {
                        int kl, kh;
                        sg_col_bounds(side, a, j0, t[0], c[0], c[1], t[1], kl, kh);
                        std::printf("%s[%d,%d,%d]", f2 ? "" : ",", j0, kl, kh);
                        f2 = false;
                    }
                    std::printf("]}");
                }
    std::printf("], \"pack\": [");
    std::mt19937 rng(7);
    first = true;
    for (int offset = 0; offset < 8; ++offset)
        for (int lim = 0; lim <= 32; lim += 1)
            for (int trial = 0; trial < 3; ++trial) {
                std::vector<unsigned char> store(offset + lim + 1);
                for (auto& v : store) v = trial == 0 ? 1 : (rng() & 1);
                const bool* row = reinterpret_cast<const bool*>(store.data()) + offset;
                std::printf("%s{\"offset\":%d,\"lim\":%d,\"bytes\":[", first ? "" : ",", offset, lim);
                first = false;
                for (int t = 0; t < lim; ++t) std::printf("%s%d", t ? "," : "", (int)store[offset + t]);
                std::printf("],\"word\":%u}", sg_pack_mask32(row, lim));
            }
    std::printf("]}\n");
    return 0;
}
