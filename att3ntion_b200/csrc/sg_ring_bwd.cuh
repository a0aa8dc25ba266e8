// Windowed single-gather backward for sm_100a ("ring" schedule).
//
// With P = softmax over the visible (j,k) pairs of query i, delta_i = dY_i . Y_i,
// dP[j][k] = sum_d dY_i[d] Vr_j[d] Vs_k[d] and gA = P o (dP - delta_i):
//
//   dS[k]  = scale * sum_{i,h,j} gA[j][k] (Q_i o R_j)      dVs[k] = sum_{i,h,j} P[j][k] (dY_i o Vr_j)
//   dQ[i]  = scale * sum_k S_k o (sum_j gA[j][k] R_j)
//
// and dR, dVr follow from the same formulas with the roles of (R, Vr) and
// (S, Vs) exchanged, because the operator is symmetric in its two key axes.
// The reference computes these in three anchored passes that each recompute the
// scores (cuda/backward.cu:415-934, roles table 2239-2247).  Here one kernel
// yields the gradients of one key side (plus dQ on request) and is launched
// twice with the sides exchanged:
//
//  * Same ring as the forward: key k occupies slot k mod 128 of the shared-memory
//    operand tiles, and -- new here -- lane k mod 128 of two FP32 accumulators in
//    tensor memory that persist across the queries and heads a CTA walks.
//  * Per (query, head), with the "own" side called (Kb, Vb) and the other (Ka, Va):
//      X^T  = Kb (Q_i o Ka)^T,  dP^T = Vb (dY_i o Va)^T        two 128x128xD MMAs
//      thread (k, column half) forms P^T = exp2(X^T c - lse) and gA^T in registers
//      and stores both to tensor memory as BF16 over the consumed score columns
//      dKb += gA^T (Q_i o Ka),  dVb += P^T (dY_i o Va)          A from tensor memory,
//                                                              B = the Hadamard tiles (MN-major)
//      dQ pass only:  W = gA^T Ka, then dQ_i = scale * sum_k Kb_k o W_k by warp shuffles.
//    The forward statistics (m, l) make P purely elementwise, so no row reduction
//    is needed here.
//  * When query i reuses slot i mod 128 the lane holding key i-128 is final for
//    this CTA: it is copied to an FP32 partial buffer and zeroed.  Neighbouring
//    query blocks write partial buffers of opposite parity and blocks are at
//    least 127 queries long, so every partial row has exactly one writer and the
//    final sum (reduce kernel below) has a fixed order: repeated calls are
//    bit-identical.
#pragma once

#include "sg_ring_fwd.cuh"

namespace sgring {

constexpr int BWD_THREADS = 256;
constexpr int BWD_MIN_BLOCK = 128;   // queries per block >= window so each partial row has one writer

struct BwdParams {
    const __nv_bfloat16* Q;          // [B,Hq,N,D]
    const __nv_bfloat16* dY;         // [B,Hq,N,D]
    const __nv_bfloat16* Y;          // [B,Hq,N,D]
    const float* m;                  // [B,Hq,N]
    const float* l;
    const __nv_bfloat16* Ka;         // other key side   [B,Hkv,N,D]
    const __nv_bfloat16* Va;
    const __nv_bfloat16* Kb;         // own key side: gradients are produced for these
    const __nv_bfloat16* Vb;
    const uint8_t* mask;             // [B,N,N] or null
    __nv_bfloat16* dQ;               // [B,Hq,N,D], written only by the WITH_DQ instantiation
    float* part_K;                   // [2][B,Hkv,N,D] FP32 partials of dKb (parity-major)
    float* part_V;                   // [2][B,Hkv,N,D] FP32 partials of dVb
    int B, Hq, Hkv, N, window, q_begin, block_len;
    float scale;
    int* status;
};

template <int D, bool WITH_DQ>
struct BwdSmem {
    static constexpr int TILE = RING * D * 2;
    static constexpr int OFF_KB = 0;
    static constexpr int OFF_VB = TILE;
    static constexpr int OFF_QP = 2 * TILE;
    static constexpr int OFF_G = 3 * TILE;
    static constexpr int OFF_KA = 4 * TILE;                       // only WITH_DQ
    static constexpr int OFF_STAGE = (WITH_DQ ? 5 : 4) * TILE;    // 2 stages x {Q, dY, Y} rows
    static constexpr int OFF_RED = OFF_STAGE + 2 * 3 * D * 2;     // 4 x D floats (dQ partials)
    static constexpr int OFF_VIS = OFF_RED + 4 * D * 4;
    static constexpr int OFF_MISC = OFF_VIS + 16;
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

template <int D, bool WITH_DQ>
__global__ void __launch_bounds__(BWD_THREADS, 1) sg_ring_bwd_kernel(const BwdParams p) {
    using L = BwdSmem<D, WITH_DQ>;
    constexpr int HD = D / 2;            // columns of d owned by one thread in the Hadamard / dQ steps
    constexpr int HCH = HD / 8;          // 16-byte chunks in that half row
    constexpr int HW = HD / 2;           // packed words in that half row
    constexpr uint32_t TMEM_COLS = 512;
    // Tensor-memory columns: scores X^T [0,128) (P^T as BF16 in [0,64)), dP^T [128,256)
    // (gA^T as BF16 in [128,192)), accumulators dKb [256,256+D) and dVb [384,384+D).
    // W = gA^T Ka (dQ pass) reuses the consumed upper halves [64,128) and [192,256).
    constexpr uint32_t C_XT = 0, C_DP = 128, C_AK = 256, C_AV = 384, C_W0 = 64, C_W1 = 192;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKb = smem + L::OFF_KB;
    uint8_t* sVb = smem + L::OFF_VB;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sG = smem + L::OFF_G;
    uint8_t* sKa = smem + L::OFF_KA;
    __nv_bfloat16* sStage = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_STAGE);
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + L::OFF_VIS);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC + 8);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 12);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = tid & (RING - 1);   // ring slot = tensor-memory lane owned by this thread
    const int half = tid >> 7;           // 0/1: which half of d (Hadamard, dQ) and of the score columns
    const int b = blockIdx.z, g = blockIdx.y;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + blockIdx.x * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const int parity = blockIdx.x & 1;

    if (warp == 0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;
    const __nv_bfloat16* gKa = p.Ka + kv_base * D;
    const __nv_bfloat16* gVa = p.Va + kv_base * D;
    const __nv_bfloat16* gKb = p.Kb + kv_base * D;
    const __nv_bfloat16* gVb = p.Vb + kv_base * D;
    float* gPartK = p.part_K + (static_cast<size_t>(parity) * p.B * p.Hkv * p.N + kv_base) * D;
    float* gPartV = p.part_V + (static_cast<size_t>(parity) * p.B * p.Hkv * p.N + kv_base) * D;

    // This thread's half row of the other side's ring slot, for the Hadamard tiles.
    uint32_t rKa[HW], rVa[HW];
    auto load_slot = [&](int key) {
        const int c0 = half * HCH;
        if (key >= 0) {
            const uint4* ka4 = reinterpret_cast<const uint4*>(gKa + static_cast<size_t>(key) * D);
            const uint4* va4 = reinterpret_cast<const uint4*>(gVa + static_cast<size_t>(key) * D);
            const uint4* kb4 = reinterpret_cast<const uint4*>(gKb + static_cast<size_t>(key) * D);
            const uint4* vb4 = reinterpret_cast<const uint4*>(gVb + static_cast<size_t>(key) * D);
#pragma unroll
            for (int c = 0; c < HCH; ++c) {
                const uint4 a = __ldg(ka4 + c0 + c), v = __ldg(va4 + c0 + c);
                rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
                rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
                *reinterpret_cast<uint4*>(sKb + sw128_offset<RING>(slot, c0 + c)) = __ldg(kb4 + c0 + c);
                *reinterpret_cast<uint4*>(sVb + sw128_offset<RING>(slot, c0 + c)) = __ldg(vb4 + c0 + c);
                if (WITH_DQ) *reinterpret_cast<uint4*>(sKa + sw128_offset<RING>(slot, c0 + c)) = a;
            }
        } else {
            const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < HCH; ++c) {
                rKa[4 * c] = rKa[4 * c + 1] = rKa[4 * c + 2] = rKa[4 * c + 3] = 0;
                rVa[4 * c] = rVa[4 * c + 1] = rVa[4 * c + 2] = rVa[4 * c + 3] = 0;
                *reinterpret_cast<uint4*>(sKb + sw128_offset<RING>(slot, c0 + c)) = z;
                *reinterpret_cast<uint4*>(sVb + sw128_offset<RING>(slot, c0 + c)) = z;
                if (WITH_DQ) *reinterpret_cast<uint4*>(sKa + sw128_offset<RING>(slot, c0 + c)) = z;
            }
        }
    };
    load_slot(ring_key(q0, slot));

    // Staged rows {Q, dY, Y} of a (query, head): stage s at sStage + s*3*D.
    const int n_iter = (q1 - q0) * G;
    auto row_index = [&](int it) {
        const int i = q0 + it / G, h = g * G + it % G;
        return (static_cast<size_t>(b) * p.Hq + h) * p.N + i;
    };
    auto stage_rows = [&](int it) {       // threads [0, 3*D/8) copy one 16-byte chunk each
        constexpr int CH = D / 8;
        if (tid < 3 * CH) {
            const int which = tid / CH, c = tid % CH;
            const __nv_bfloat16* src = (which == 0 ? p.Q : which == 1 ? p.dY : p.Y) + row_index(it) * D;
            const uint32_t dst = smem_u32(sStage + ((it & 1) * 3 + which) * D) + c * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                         "l"(reinterpret_cast<const uint4*>(src) + c)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_rows(0);
    asm volatile("cp.async.wait_all;" ::: "memory");

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tl = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);   // this warp's lane quarter

    // Zero the two persistent accumulators: half 0 clears dKb, half 1 clears dVb.
    {
        uint32_t z[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) z[t] = 0;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_st32(tl + (half ? C_AV : C_AK) + c * 32, z);
        tmem_wait_st();
    }

    // Copies lane `slot`'s accumulator row to the partial buffers (row `key`) and,
    // unless this is the final drain, zeroes it.  Runs on the two warps that own
    // the lane quarter `quarter`; warp-uniform control flow around the collective
    // tensor-memory accesses.
    auto flush = [&](int quarter, int only_lane /* -1: all lanes */, int i_ref, bool rezero) {
        if ((warp & 3) != quarter) return;
        const uint32_t col = half ? C_AV : C_AK;
        float* dst_base = half ? gPartV : gPartK;
        const float mul = half ? 1.0f : p.scale;
        const int key = ring_key(i_ref, slot);
        const bool mine = (only_lane < 0 || lane == only_lane) && key >= 0;
        uint32_t a[32];
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(tl + col + c * 32, a);
            tmem_wait_ld();
            if (mine) {
                float4* dst = reinterpret_cast<float4*>(dst_base + static_cast<size_t>(key) * D + c * 32);
#pragma unroll
                for (int t = 0; t < 8; ++t)
                    dst[t] = make_float4(mul * __uint_as_float(a[4 * t]), mul * __uint_as_float(a[4 * t + 1]),
                                         mul * __uint_as_float(a[4 * t + 2]), mul * __uint_as_float(a[4 * t + 3]));
            }
            if (rezero) {
                if (only_lane < 0 || lane == only_lane) {
#pragma unroll
                    for (int t = 0; t < 32; ++t) a[t] = 0;
                }
                tmem_st32(tl + col + c * 32, a);
            }
        }
        if (rezero) tmem_wait_st();
    };

    const uint32_t idesc_s = make_idesc_bf16(RING, RING, 0, 0);     // score-shaped, both operands K-major
    const uint32_t idesc_acc = make_idesc_bf16(RING, D, 0, 1);      // A in tensor memory, B MN-major, N = D
    const uint32_t idesc_w = make_idesc_bf16(RING, 64, 0, 1);       // W halves, N = 64
    const uint32_t aKb = smem_u32(sKb), aVb = smem_u32(sVb), aQp = smem_u32(sQp), aG = smem_u32(sG),
                   aKa = smem_u32(sKa);
    const float c2 = p.scale * LOG2E;
    uint32_t phase = 0;
    bool failed = false;

    int it = 0;
    for (int i = q0; i < q1 && !failed; ++i) {
        // --- slide the window ---------------------------------------------------
        if (i > q0) {
            const int s = i & (RING - 1);
            flush(s >> 5, s & 31, i - 1, true);      // slot s still maps to key i-128 under query i-1
            if (slot == s) load_slot(i);
        }
        bool my_vis;
        {
            const int key = ring_key(i, slot);
            my_vis = key >= 0 && key > i - p.window;
            if (my_vis && p.mask) my_vis = p.mask[(static_cast<size_t>(b) * p.N + i) * p.N + key] != 0;
            const uint32_t w = __ballot_sync(0xFFFFFFFFu, my_vis);
            if (lane == 0 && warp < 4) sVis[warp] = w;
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        const uint32_t vw0 = sVis[0], vw1 = sVis[1], vw2 = sVis[2], vw3 = sVis[3];
        const int n_vis = __popc(vw0) + __popc(vw1) + __popc(vw2) + __popc(vw3);
        const bool all_vis = n_vis == RING;

        for (int hh = 0; hh < G && !failed; ++hh, ++it) {
            const size_t row = row_index(it);
            if (it + 1 < n_iter) stage_rows(it + 1);
            const float m_i = __ldg(p.m + row), l_i = __ldg(p.l + row);
            const __nv_bfloat16* stQ = sStage + (it & 1) * 3 * D;
            const __nv_bfloat16* stdY = stQ + D;
            const __nv_bfloat16* stY = stQ + 2 * D;

            if (n_vis == 0 || !(l_i > 0.f)) {
                // No visible pair: every gradient contribution of this query is zero.
                if (WITH_DQ && tid < D) p.dQ[row * D + tid] = __float2bfloat16(0.f);
                asm volatile("cp.async.wait_all;" ::: "memory");
                __syncthreads();
                continue;
            }

            // delta = sum_d dY[d] * Y[d], the same value in every warp
            float delta = 0.f;
#pragma unroll
            for (int t = 0; t < D / 32; ++t)
                delta += __bfloat162float(stdY[lane + 32 * t]) * __bfloat162float(stY[lane + 32 * t]);
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) delta += __shfl_xor_sync(0xFFFFFFFFu, delta, o);
            const float lse2 = m_i * LOG2E + __log2f(l_i);

            // --- Hadamard tiles: Qp[j] = Q_i o Ka_j, Gt[j] = dY_i o Va_j (this thread: half a row)
            {
                const uint4* q4 = reinterpret_cast<const uint4*>(stQ) + half * HCH;
                const uint4* y4 = reinterpret_cast<const uint4*>(stdY) + half * HCH;
#pragma unroll
                for (int c = 0; c < HCH; ++c) {
                    const uint4 q = q4[c], y = y4[c];
                    uint4 o, gq;
                    o.x = mul_bf16x2(q.x, rKa[4 * c]);      gq.x = mul_bf16x2(y.x, rVa[4 * c]);
                    o.y = mul_bf16x2(q.y, rKa[4 * c + 1]);  gq.y = mul_bf16x2(y.y, rVa[4 * c + 1]);
                    o.z = mul_bf16x2(q.z, rKa[4 * c + 2]);  gq.z = mul_bf16x2(y.z, rVa[4 * c + 2]);
                    o.w = mul_bf16x2(q.w, rKa[4 * c + 3]);  gq.w = mul_bf16x2(y.w, rVa[4 * c + 3]);
                    *reinterpret_cast<uint4*>(sQp + sw128_offset<RING>(slot, half * HCH + c)) = o;
                    *reinterpret_cast<uint4*>(sG + sw128_offset<RING>(slot, half * HCH + c)) = gq;
                }
            }
            fence_async_smem();
            tc_fence_before();
            __syncthreads();                                                   // B1
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * (RING * 128) + (kk & 3) * 32;
                    umma_ss(tmem_base + C_XT, make_smem_desc(aKb + off, 16, 1024, SWIZZLE_128B),
                            make_smem_desc(aQp + off, 16, 1024, SWIZZLE_128B), idesc_s, kk > 0);
                }
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * (RING * 128) + (kk & 3) * 32;
                    umma_ss(tmem_base + C_DP, make_smem_desc(aVb + off, 16, 1024, SWIZZLE_128B),
                            make_smem_desc(aG + off, 16, 1024, SWIZZLE_128B), idesc_s, kk > 0);
                }
                umma_commit(bar);
                if (!mbar_wait(bar, phase)) *sFail = 1;
            }
            phase ^= 1;
            __syncthreads();                                                   // B2
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            // --- P^T and gA^T for this thread's (lane k, 32-column chunk) in two rounds.  Round r
            //     covers chunks 2r (half 0) and 2r+1 (half 1); their BF16 results land on columns
            //     that both halves have finished reading, hence the barrier inside the round.
            const bool single = n_vis == 1;     // one visible key: score gradients are exactly zero
#pragma unroll 1
            for (int rd = 0; rd < 2; ++rd) {
                const int c = 2 * rd + half;
                uint32_t x[32], dp[32], pk[16], gk[16];
                tmem_ld32(tl + C_XT + c * 32, x);
                tmem_ld32(tl + C_DP + c * 32, dp);
                tmem_wait_ld();
                const uint32_t cw = my_vis ? (rd == 0 ? (half ? vw1 : vw0) : (half ? vw3 : vw2)) : 0u;
#pragma unroll
                for (int t = 0; t < 32; t += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(x[t]), c2, -lse2));
                    float p1 = fast_exp2(fmaf(__uint_as_float(x[t + 1]), c2, -lse2));
                    if (!all_vis) {
                        if (!((cw >> t) & 1u)) p0 = 0.f;
                        if (!((cw >> (t + 1)) & 1u)) p1 = 0.f;
                    }
                    float g0 = p0 * (__uint_as_float(dp[t]) - delta);
                    float g1 = p1 * (__uint_as_float(dp[t + 1]) - delta);
                    if (single) { g0 = 0.f; g1 = 0.f; }
                    pk[t >> 1] = pack_bf16x2(p0, p1);
                    gk[t >> 1] = pack_bf16x2(g0, g1);
                }
                tc_fence_before();
                __syncthreads();
                tc_fence_after();
                tmem_st16(tl + C_XT + c * 16, pk);
                tmem_st16(tl + C_DP + c * 16, gk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncthreads();                                                   // B3
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < RING / 16; ++kk)      // dKb += gA^T . Qp
                    umma_ts(tmem_base + C_AK, tmem_base + C_DP + kk * 8,
                            make_smem_desc(aQp + kk * 2048, RING * 128, 1024, SWIZZLE_128B), idesc_acc, 1);
#pragma unroll
                for (int kk = 0; kk < RING / 16; ++kk)      // dVb += P^T . Gt
                    umma_ts(tmem_base + C_AV, tmem_base + C_XT + kk * 8,
                            make_smem_desc(aG + kk * 2048, RING * 128, 1024, SWIZZLE_128B), idesc_acc, 1);
                if (WITH_DQ) {
#pragma unroll
                    for (int dh = 0; dh < D / 64; ++dh)     // W[:, 64 dh ..] = gA^T . Ka
#pragma unroll
                        for (int kk = 0; kk < RING / 16; ++kk)
                            umma_ts(tmem_base + (dh ? C_W1 : C_W0), tmem_base + C_DP + kk * 8,
                                    make_smem_desc(aKa + dh * (RING * 128) + kk * 2048, RING * 128, 1024,
                                                   SWIZZLE_128B),
                                    idesc_w, kk > 0);
                }
                umma_commit(bar);
                if (!mbar_wait(bar, phase)) *sFail = 1;
            }
            phase ^= 1;
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();                                                   // B4
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            if (WITH_DQ) {
                // dQ[d] = scale * sum_k Kb_k[d] * W[k][d]; this thread: lane k, d in its half.
                // D = 128: half h reads W columns of d-block h.  D = 64: both halves share block 0.
                const uint32_t wcol = (D == 128) ? (half ? C_W1 : C_W0) : (C_W0 + half * 32);
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t u[32];
                    float v[32];
                    tmem_ld32(tl + wcol + c * 32, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 kb =
                            *reinterpret_cast<const uint4*>(sKb + sw128_offset<RING>(slot, half * HCH + c * 4 + q));
                        const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 kf = unpack_bf16x2(w4[e]);
                            v[q * 8 + 2 * e] = kf.x * __uint_as_float(u[q * 8 + 2 * e]);
                            v[q * 8 + 2 * e + 1] = kf.y * __uint_as_float(u[q * 8 + 2 * e + 1]);
                        }
                    }
                    const float s = warp_transpose_sum(v, lane);
                    sRed[(warp & 3) * D + half * HD + c * 32 + lane] = s;
                }
                tc_fence_before();
                __syncthreads();                                               // B5
                if (tid < D)
                    p.dQ[row * D + tid] =
                        __float2bfloat16(p.scale * (sRed[tid] + sRed[D + tid] + sRed[2 * D + tid] + sRed[3 * D + tid]));
            }
        }
    }
    // Drain: every slot still holds a key of (q1 - 129, q1 - 1].
    if (!failed) {
#pragma unroll 1
        for (int quarter = 0; quarter < 4; ++quarter) flush(quarter, -1, q1 - 1, false);
    }
    if (failed && tid == 0) atomicExch(p.status, 2);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Sums the parity partials of one key side into BF16 outputs.  Row k of batch b,
// KV head g was written by the query blocks that contain a query in [k, k+127]
// (clipped to [q_begin, N)); consecutive blocks use opposite parities, so at
// most one block per parity contributes and the order of the sum is fixed.
struct ReduceParams {
    const float* part_K;
    const float* part_V;
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    int rows;            // B * Hkv
    int N, D, q_begin, block_len, nblk;
};

__global__ void sg_bwd_reduce_kernel(const ReduceParams p) {
    const int chunks = p.D / 4;
    const size_t total = static_cast<size_t>(p.rows) * p.N * chunks;
    const size_t plane = static_cast<size_t>(p.rows) * p.N * p.D;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(idx % chunks);
        const size_t rk = idx / chunks;
        const int k = static_cast<int>(rk % p.N);
        const int q_lo = max(k, p.q_begin), q_hi = min(k + RING - 1, p.N - 1);
        float4 sk = make_float4(0.f, 0.f, 0.f, 0.f), sv = sk;
        if (q_lo <= q_hi) {
            const int b_lo = (q_lo - p.q_begin) / p.block_len, b_hi = (q_hi - p.q_begin) / p.block_len;
            for (int blk = b_lo; blk <= b_hi; ++blk) {
                const size_t off = static_cast<size_t>(blk & 1) * plane + rk * p.D + c * 4;
                const float4 a = *reinterpret_cast<const float4*>(p.part_K + off);
                const float4 v = *reinterpret_cast<const float4*>(p.part_V + off);
                sk.x += a.x; sk.y += a.y; sk.z += a.z; sk.w += a.w;
                sv.x += v.x; sv.y += v.y; sv.z += v.z; sv.w += v.w;
            }
        }
        uint2 ok, ov;
        ok.x = pack_bf16x2(sk.x, sk.y); ok.y = pack_bf16x2(sk.z, sk.w);
        ov.x = pack_bf16x2(sv.x, sv.y); ov.y = pack_bf16x2(sv.z, sv.w);
        *reinterpret_cast<uint2*>(p.dK + rk * p.D + c * 4) = ok;
        *reinterpret_cast<uint2*>(p.dV + rk * p.D + c * 4) = ov;
    }
}

}  // namespace sgring
