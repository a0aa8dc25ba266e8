// Pieces shared by the windowed single-gather kernels for sm_100a: the ring convention, the
// role-specialised CTA skeleton (thread counts, register budgets), bounded mbarrier waits and the
// warp-level reductions.
#pragma once

#include "sm100_ptx.cuh"

namespace sgring {

using namespace sm100;

constexpr int RING = 128;          // keys resident per CTA = maximum window
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_INF_F = -1e30f;   // statistics value of a query with no visible pair

// Key index held by ring slot `slot` while query i is processed: the unique
// index congruent to slot (mod 128) in (i - 128, i].
__device__ __forceinline__ int ring_key(int i, int slot) { return i - ((i - slot) & (RING - 1)); }

// Sum over the 32 lanes of a warp of 32 per-lane values; lane L ends up with the
// total of element L in v[0].  31 shuffles.
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int k = 0; k < o; ++k) {
            const float send = up ? v[k] : v[k + o];
            const float keep = up ? v[k + o] : v[k];
            v[k] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
        }
    }
    return v[0];
}

constexpr int PIPE_E_THREADS = 256;
constexpr int PIPE_H_THREADS = 128;
// Four full warpgroups: E (2), H (1) and one whose first warp issues the MMAs while the
// other three only hand their registers to the working roles (setmaxnreg below).
constexpr int PIPE_THREADS = PIPE_E_THREADS + PIPE_H_THREADS + 128;

template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// One arrival per warp: the lanes' earlier writes are ordered before lane 0's releasing
// arrive by the warp barrier.  256 per-thread arrivals on one barrier word serialise into
// more than a thousand cycles per hand-off; eight do not.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// Bounded wait on an mbarrier phase.  try_wait parks the thread in hardware until the phase
// completes or a system time limit passes.  Measured alternatives on this part, same kernels:
// all threads spinning on test_wait pulled the SM clock from 1.9 to 1.3 GHz under the power
// cap (2x the run time); one polling lane per warp with __nanosleep(20) between polls was
// 2.3x slower still (the sleep is far coarser than its argument); one polling lane with the
// result shuffled to the others costs 245 cycles on a complete phase against 50-90 for all
// 32 lanes waiting together (the divergent branch, not the barrier, is what costs).  On a
// complete phase test_wait and try_wait without a time hint return in ~50 cycles, try_wait
// with a hint in ~90: the loop therefore gives no hint (forward 4.42 -> 4.27 ms, backward
// 11.07 -> 10.68 ms on B4 Hq8 N8192), and TEST_FIRST puts a plain test in front of it, which
// gained another 0.1 ms in the forward and lost as much in the backward.  The iteration
// count bounds the total wait: a poll of a pending phase returns after the system limit,
// measured at 7.8 k cycles (4 us), so a wait gives up after about 2 s; the loop also leaves
// when another thread has raised the CTA's failure flag.
template <bool TEST_FIRST = false>
__device__ __forceinline__ bool pipe_wait(uint64_t* bar, uint32_t parity, volatile int* fail, int code = 1) {
    const uint32_t addr = smem_u32(bar);
    if (TEST_FIRST) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
#pragma unroll 1
    for (uint32_t it = 0; it < (1u << 19); ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((it & 15u) == 15u && *fail) return false;
    }
    *fail = code;      // which wait gave up (reported through the status word)
    return false;
}

// A caller's visibility mask comes as bytes ([B,N,N], non-zero = visible) or as packed words ([B,N,ceil(N/32)],
// bit t of word c = key 32 c + t: the form of the reference's mask metadata, cuda/shared_kv/shared_mask_metadata.cuh:8-31,
// 32 times less to read); MaskRow is one query's row of either, MaskView the batch's.
struct MaskRow {
    const uint8_t* bytes;
    const uint32_t* words;
    __device__ __forceinline__ bool any() const { return bytes != nullptr || words != nullptr; }
    __device__ __forceinline__ bool at(int key) const {
        return words ? ((__ldg(words + (key >> 5)) >> (key & 31)) & 1u) != 0 : bytes[key] != 0;
    }
};
struct MaskView {
    const uint8_t* bytes;
    const uint32_t* words;
    int N, NW;
    __device__ __forceinline__ bool any() const { return bytes != nullptr || words != nullptr; }
    __device__ __forceinline__ MaskRow row(int i) const {
        return MaskRow{bytes ? bytes + static_cast<size_t>(i) * N : nullptr,
                       words ? words + static_cast<size_t>(i) * NW : nullptr};
    }
};
__device__ __forceinline__ MaskView mask_view(const uint8_t* bytes, const uint32_t* words, int b, int N) {
    const int NW = (N + 31) / 32;
    return MaskView{bytes ? bytes + static_cast<size_t>(b) * N * N : nullptr,
                    words ? words + static_cast<size_t>(b) * N * NW : nullptr, N, NW};
}

// Residual of a packed BF16 product: with hi = bf16x2(a * b) (round to nearest), returns bf16x2(a * b - hi).  The
// product of two BF16 numbers has at most 16 significant bits, so it is exact in FP32, and so is the difference,
// which has at most 8 significant bits and is therefore exact in BF16 (barring underflow): hi + lo carries the
// product without rounding.  This is the split the reference prototyped as its "compensated" path
// (docs/KERNEL_HISTORY.md:22: high + residual parts of each BF16 product).
__device__ __forceinline__ uint32_t mul_residual_bf16x2(uint32_t a, uint32_t b, uint32_t hi) {
    const float2 fa = unpack_bf16x2(a), fb = unpack_bf16x2(b), fh = unpack_bf16x2(hi);
    return pack_bf16x2(fa.x * fb.x - fh.x, fa.y * fb.y - fh.y);
}

// Memory layout of the [B,H,N,D] operands.  0: B,H,N,D contiguous (the reference's, cuda/forward.cu:1609-1631).
// 1: B,N,H,D contiguous -- what a projection x W gives before the head split is permuted and copied
// (att3ntion/_autograd.py:349-363 does that copy for every operand of every call).  Statistics are [B,H,N] in
// both.  A row is named by its index in the statistics, r = (b*H + head)*N + i; RowAddr turns that into the
// element offset of the row and into the (x, y) coordinates of a 2-D tensor map over the same memory
// (layout 0: [B*H*N, D]; layout 1: [B*N, H*D] with the head as a column offset).
struct RowAddr {
    int bnhd, H, N, D;
    __device__ __forceinline__ size_t elem(size_t r) const {
        if (!bnhd) return r * D;
        const size_t bh = r / N;
        const int i = static_cast<int>(r - bh * N), head = static_cast<int>(bh % H);
        return ((bh / H * N + i) * H + head) * static_cast<size_t>(D);
    }
    __device__ __forceinline__ void tma(size_t r, int& x, int& y) const {
        if (!bnhd) { x = 0; y = static_cast<int>(r); return; }
        const size_t bh = r / N;
        const int i = static_cast<int>(r - bh * N), head = static_cast<int>(bh % H);
        x = head * D;
        y = static_cast<int>(bh / H * N + i);
    }
    // elements between the rows of consecutive positions of one (batch, head)
    __device__ __forceinline__ size_t step() const { return bnhd ? static_cast<size_t>(H) * D : D; }
};

// Visibility of the 128 ring slots for query i as four ballot words; every warp
// computes the same words (lane L looks at slots L, 32+L, 64+L, 96+L).
__device__ __forceinline__ void ring_visibility(const MaskRow mask_row, int i, int window, int lane, uint32_t (&vw)[4]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int key = ring_key(i, q * 32 + lane);
        bool v = key >= 0 && key > i - window;
        if (v && mask_row.any()) v = mask_row.at(key);
        vw[q] = __ballot_sync(0xFFFFFFFFu, v);
    }
}

// Sum over the 32 lanes of a warp of 32 per-lane values given as two halves (va: values 0-15,
// vb: values 16-31); lane L ends up with the total of value L.  Same exchange network as
// warp_transpose_sum, with the first stage folding the two halves.
__device__ __forceinline__ float warp_transpose_sum_2x16(float (&va)[16], float (&vb)[16], int lane) {
    {
        const bool up = (lane & 16) != 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float send = up ? va[k] : vb[k];
            const float keep = up ? vb[k] : va[k];
            va[k] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 16);
        }
    }
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int k = 0; k < o; ++k) {
            const float send = up ? va[k] : va[k + o];
            const float keep = up ? va[k + o] : va[k];
            va[k] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
        }
    }
    return va[0];
}

// The same lane sum with the first four exchange stages on packed BF16 pairs (adjacent values of a
// lane share a register), the last one and the result in FP32: 80 instead of ~125 instructions.  The
// partial sums are rounded to BF16 at each of the four packed stages (relative 2^-9 each), which is the
// precision of the MMA operands these sums are built from; the gates leave an order of magnitude of room.
// w[k] holds this lane's values 2k and 2k+1 as a BF16 pair.
__device__ __forceinline__ float warp_transpose_sum_words(uint32_t (&w)[16], int lane) {
    // stage o (in values) exchanges value v with v ^ o across lanes l and l ^ o; in packed registers that is
    // register r with r ^ (o/2) for o >= 2
#pragma unroll
    for (int o = 16; o >= 2; o >>= 1) {
        const bool up = (lane & o) != 0;
        const int h = o >> 1;                                  // packed registers per half
#pragma unroll
        for (int k = 0; k < h; ++k) {
            const uint32_t send = up ? w[k] : w[k + h];
            const uint32_t keep = up ? w[k + h] : w[k];
            const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, send, o);
            __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&keep);
            __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&got);
            __nv_bfloat162 c = __hadd2(a, b);
            w[k] = *reinterpret_cast<uint32_t*>(&c);
        }
    }
    // one register left: the two values of this lane pair; even lanes finish the first, odd lanes the second
    const float2 mine = unpack_bf16x2(w[0]);
    const bool odd = (lane & 1) != 0;
    const float send = odd ? mine.x : mine.y;
    const float keep = odd ? mine.y : mine.x;
    return keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
}

// The same from FP32 values: one rounding to BF16 first.
__device__ __forceinline__ float warp_transpose_sum_2x16_packed(const float (&va)[16], const float (&vb)[16], int lane) {
    uint32_t w[16];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        w[k] = pack_bf16x2(va[2 * k], va[2 * k + 1]);           // values 2k, 2k+1
        w[8 + k] = pack_bf16x2(vb[2 * k], vb[2 * k + 1]);       // values 16+2k, 16+2k+1
    }
    return warp_transpose_sum_words(w, lane);
}

}  // namespace sgring
