// Dense anchored gather, forward, for sm_100a.
//
//   Y[a] = sum_{j,k} softmax_{(j,k)}( scale * sum_d A_a[d] Rw_j[d] C_k[d] ) Vrow[j] o Vcol[k]
//
// for an "anchor" tensor A and two key-side tensors Rw ("rows") and C ("cols"),
// every key a candidate, visibility given by a [B,N,N] mask (pair (j,k) is live for
// anchor a iff mask[b,a,j] and mask[b,a,k]) and by a valid length.  This one
// operator serves the reference's anchored tensor-core gather with its three role
// bindings (cuda/forward.cu:108-477 and the role table at its launcher): Y_q uses
// (A,Rw,C) = (Q,R,S), Y_r = (R,Q,S), Y_s = (S,Q,R); and the un-windowed
// single_gather_forward (cuda/forward.cu:1666-1719) is the first binding alone.
//
// Schedule: a CTA owns a group of anchors of one (batch, head).  It walks the
// 128x128 (row tile, col tile) grid; the col tile (C, Vcol) is staged once per tile
// in shared memory in the 128-byte swizzle, the row tile (Rw, Vrow) lives in
// registers, one row per thread.  For every anchor of the group the tile is
// processed exactly like one (query, head) of the windowed kernel
// (sg_ring_fwd.cuh): Hadamard tile -> score MMA -> per-row softmax -> value MMA with
// P read from tensor memory -> shuffle collapse; the per-tile result is merged into
// the anchor's running (max, sum, Y) state in shared memory with the usual
// log-sum-exp rescaling.  Head dims below 64 are zero-padded to 64 in the operand
// tiles (the padding contributes nothing to either contraction).
#pragma once

#include "sg_ring_fwd.cuh"

namespace agdense {

using namespace sm100;
using sgring::warp_transpose_sum;
using sgring::LOG2E;
using sgring::NEG_INF_F;

constexpr int TILE = 128;
constexpr int NTHREADS = 128;
constexpr int MAX_GROUP = 16;       // anchors per CTA

struct FwdParams {
    const __nv_bfloat16* A;         // anchor   [B,H,NA,D]
    const __nv_bfloat16* Rw;        // rows     [B,H,NR,D]
    const __nv_bfloat16* C;         // cols     [B,H,NC,D]
    const __nv_bfloat16* Vrow;      // [B,H,NR,D]
    const __nv_bfloat16* Vcol;      // [B,H,NC,D]
    const uint8_t* mask;            // [B,N,N] or null (then NA = NR = NC = N); row index = anchor
    __nv_bfloat16* Y;               // [B,H,NA,D]
    float* m;                       // [B,H,NA]
    float* l;
    // Lengths of the three index axes and how many leading entries of each are real (the rest is padding that stays
    // out of every softmax; 0 or > length: all).  The reference's gather takes the same five numbers
    // (cuda/forward.cu:1436-1452: n_anchor, n_rows, rows_valid, n_cols, cols_valid); a_valid only matters to the scatter form.
    int B, H, NA, NR, NC, D, a_valid, r_valid, c_valid, group;
    float scale;
    int* status;
    // Scatter form (SC kernels only): statistics of the softmaxes anchored at the row index and at the col index
    const float* m_row; const float* l_row;
    const float* m_col; const float* l_col;
};

template <int DP>
struct FwdSmem {
    static constexpr int TILE_BYTES = TILE * DP * 2;
    static constexpr int OFF_C = 0;
    static constexpr int OFF_VC = TILE_BYTES;
    static constexpr int OFF_QP = 2 * TILE_BYTES;
    static constexpr int OFF_STATE = 3 * TILE_BYTES;                       // MAX_GROUP x (DP + 4) floats
    static constexpr int OFF_RED = OFF_STATE + MAX_GROUP * (DP + 4) * 4;   // 4 x (DP + 4) floats
    static constexpr int OFF_MPART = OFF_RED + 4 * (DP + 4) * 4;
    static constexpr int OFF_VIS = OFF_MPART + 16;                         // 4 row words + 4 col words
    static constexpr int OFF_MISC = OFF_VIS + 32;
    static constexpr int OFF_COLL = OFF_MISC + 16;                         // scatter form: 128 col constants
    static constexpr int BYTES = OFF_COLL + TILE * 4;
    static constexpr int ALLOC = BYTES + 1024;
};

// Loads row `idx` (D valid BF16, zero-padded to DP) of a [N][D] matrix as packed words.
template <int DP>
__device__ __forceinline__ void load_row_padded(const __nv_bfloat16* base, int idx, int N, int D, uint32_t (&r)[DP / 2]) {
#pragma unroll
    for (int c = 0; c < DP / 8; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (idx < N && c * 8 < D) v = __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(idx) * D) + c);
        r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
    }
}

// SC = true turns the gather into one scatter output of the three-gather operator
// (cpp/torch_reference.cpp:51-54, cuda/forward.cu:941-1249): with the output index as the anchor a and the
// two other indices as rows u and cols v,
//   out[a] = sum_{u,v} W[a,u,v] Vrow[u] o Vcol[v],   W = Pu Pv = exp(2 x - LSE_u[u] - LSE_v[v]),
// Pu being the softmax anchored at u (taken over (a, v)) and Pv the one anchored at v, both finished by
// earlier gathers whose statistics arrive as (m_row, l_row) and (m_col, l_col).  The exponent is <= 0 because
// each LSE is taken over a set that contains the cell, so there is no running maximum and no normalisation:
// the tile loop just adds.  A cell is live iff anchor u sees a and v and anchor v sees a and u
// (mask[u][a], mask[u][v], mask[v][a], mask[v][u]) and all three indices are below the valid length.
template <int DP, bool SC = false>
__global__ void __launch_bounds__(NTHREADS, 2) ag_dense_fwd_kernel(const FwdParams p) {
    using L = FwdSmem<DP>;
    constexpr int CH = DP / 8, DW = DP / 2;
    constexpr uint32_t TMEM_COLS = 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sC = smem + L::OFF_C;
    uint8_t* sVc = smem + L::OFF_VC;
    uint8_t* sQp = smem + L::OFF_QP;
    float* sState = reinterpret_cast<float*>(smem + L::OFF_STATE);
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    float* sMpart = reinterpret_cast<float*>(smem + L::OFF_MPART);
    uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + L::OFF_VIS);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC + 8);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 12);
    float* sColL = reinterpret_cast<float*>(smem + L::OFF_COLL);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t issuer = elect_one();     // one lane per warp; warp 0 predicates its MMAs on it
    const int b = blockIdx.z, h = blockIdx.y;
    const int N = p.NA, D = p.D;                 // N: the mask's side (a mask needs equal lengths)
    const int n_rows = (p.r_valid > 0 && p.r_valid < p.NR) ? p.r_valid : p.NR;   // rows at or past this index are padding
    const int n_cols = (p.c_valid > 0 && p.c_valid < p.NC) ? p.c_valid : p.NC;
    const int n_anch = (p.a_valid > 0 && p.a_valid < p.NA) ? p.a_valid : p.NA;
    const int a0 = blockIdx.x * p.group;
    const int a1 = min(a0 + p.group, SC ? n_anch : p.NA);    // padded anchors take no part in a scatter sum
    if (a0 >= a1) return;

    if (warp == 0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        *sFail = 0;
    }
    // running state per anchor of the group: [0, DP) Y accumulator, [DP] max (raw score units), [DP+1] sum
    for (int t = tid; t < MAX_GROUP * (DP + 4); t += NTHREADS) sState[t] = 0.f;
    if (tid < MAX_GROUP) sState[tid * (DP + 4) + DP] = -INFINITY;

    const size_t bh = (static_cast<size_t>(b) * p.H + h) * p.NA;        // anchor-indexed arrays
    const size_t bh_r = (static_cast<size_t>(b) * p.H + h) * p.NR, bh_c = (static_cast<size_t>(b) * p.H + h) * p.NC;
    const __nv_bfloat16* gA = p.A + bh * D;
    const __nv_bfloat16* gRw = p.Rw + bh_r * D;
    const __nv_bfloat16* gC = p.C + bh_c * D;
    const __nv_bfloat16* gVrow = p.Vrow + bh_r * D;
    const __nv_bfloat16* gVcol = p.Vcol + bh_c * D;
    const uint8_t* mask_b = p.mask ? p.mask + static_cast<size_t>(b) * N * N : nullptr;

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tX = tmem_base + lane_field, tU = tmem_base + lane_field + 128;
    const uint32_t idesc_x = make_idesc_bf16(TILE, TILE, 0, 0);
    const uint32_t idesc_u = make_idesc_bf16(TILE, DP, 0, 1);
    const uint64_t dQp = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);
    const uint64_t dC = make_smem_desc(smem_u32(sC), 16, 1024, SWIZZLE_128B);
    const uint64_t dVcM = make_smem_desc(smem_u32(sVc), TILE * 128, 1024, SWIZZLE_128B);
    const float c2 = p.scale * LOG2E;
    uint32_t phase = 0;
    bool failed = false;

    const int row_tiles = (n_rows + TILE - 1) / TILE, col_tiles = (n_cols + TILE - 1) / TILE;
    for (int jb = 0; jb < row_tiles && !failed; ++jb) {
        uint32_t rRw[DW], rVr[DW];
        const int jrow = jb * TILE + tid;
        load_row_padded<DP>(gRw, jrow, n_rows, D, rRw);
        load_row_padded<DP>(gVrow, jrow, n_rows, D, rVr);
        // scatter form: LSE (log2 units) of the softmax anchored at this thread's row; an anchor without any
        // visible cell (l = 0) or a padded one gets a value that makes every weight vanish
        float lse_row = 1e30f;
        if (SC && jrow < n_rows) {
            const float lu = __ldg(p.l_row + bh_r + jrow);
            if (lu > 0.f) lse_row = __ldg(p.m_row + bh_r + jrow) * LOG2E + __log2f(lu);
        }
        for (int kb = 0; kb < col_tiles && !failed; ++kb) {
            // stage the col tile; every MMA that read the previous one has been waited for
            {
                uint32_t t[DW];
                const int krow = kb * TILE + tid;
                load_row_padded<DP>(gC, krow, n_cols, D, t);
#pragma unroll
                for (int c = 0; c < CH; ++c)
                    *reinterpret_cast<uint4*>(sC + sw128_offset<TILE>(tid, c)) =
                        make_uint4(t[4 * c], t[4 * c + 1], t[4 * c + 2], t[4 * c + 3]);
                load_row_padded<DP>(gVcol, krow, n_cols, D, t);
#pragma unroll
                for (int c = 0; c < CH; ++c)
                    *reinterpret_cast<uint4*>(sVc + sw128_offset<TILE>(tid, c)) =
                        make_uint4(t[4 * c], t[4 * c + 1], t[4 * c + 2], t[4 * c + 3]);
            }
            // scatter form: col constants of the tile, and the pairs (u, v) in which each anchor sees the other
            uint32_t pw0 = 0xFFFFFFFFu, pw1 = 0xFFFFFFFFu, pw2 = 0xFFFFFFFFu, pw3 = 0xFFFFFFFFu;
            if (SC) {
                const int krow = kb * TILE + tid;
                float lc = 1e30f;
                if (krow < n_cols) {
                    const float lv = __ldg(p.l_col + bh_c + krow);
                    if (lv > 0.f) lc = __ldg(p.m_col + bh_c + krow) * LOG2E + __log2f(lv);
                }
                sColL[tid] = lc;
                if (mask_b) {
                    uint32_t w[4] = {0, 0, 0, 0};
                    if (jrow < n_rows) {
                        for (int t = 0; t < TILE; ++t) {
                            const int v = kb * TILE + t;
                            if (v < n_cols && mask_b[static_cast<size_t>(jrow) * N + v] != 0 &&
                                mask_b[static_cast<size_t>(v) * N + jrow] != 0)
                                w[t >> 5] |= 1u << (t & 31);
                        }
                    }
                    pw0 = w[0]; pw1 = w[1]; pw2 = w[2]; pw3 = w[3];
                }
            }
            fence_async_smem();
            for (int a = a0; a < a1 && !failed; ++a) {
                // visibility of this tile's rows and cols from anchor a
                {
                    const int krow = kb * TILE + tid;
                    bool vr = jrow < n_rows, vc = krow < n_cols;
                    if (mask_b && SC) {
                        // the anchors of the two softmaxes are the row and the col: each must see a
                        if (vr) vr = mask_b[static_cast<size_t>(jrow) * N + a] != 0;
                        if (vc) vc = mask_b[static_cast<size_t>(krow) * N + a] != 0;
                    } else if (mask_b) {
                        const uint8_t* mrow = mask_b + static_cast<size_t>(a) * N;
                        if (vr) vr = mrow[jrow] != 0;
                        if (vc) vc = mrow[krow] != 0;
                    }
                    const uint32_t wr = __ballot_sync(0xFFFFFFFFu, vr), wc = __ballot_sync(0xFFFFFFFFu, vc);
                    if (lane == 0) { sVis[warp] = wr; sVis[4 + warp] = wc; }
                }
                __syncthreads();
                const uint32_t vr_any = sVis[0] | sVis[1] | sVis[2] | sVis[3];
                const uint32_t vc0 = sVis[4], vc1 = sVis[5], vc2 = sVis[6], vc3 = sVis[7];
                const bool my_vis = (sVis[warp] >> lane) & 1u;
                const bool all_cols = (vc0 & vc1 & vc2 & vc3) == 0xFFFFFFFFu;
                if (vr_any == 0 || (vc0 | vc1 | vc2 | vc3) == 0) {
                    __syncthreads();          // sVis is rewritten by the next anchor
                    continue;
                }
                // --- Hadamard tile from the anchor row -----------------------------------------
                {
                    uint32_t q[DW];
                    load_row_padded<DP>(gA, a, p.NA, D, q);
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        uint4 o;
                        o.x = mul_bf16x2(q[4 * c], rRw[4 * c]);
                        o.y = mul_bf16x2(q[4 * c + 1], rRw[4 * c + 1]);
                        o.z = mul_bf16x2(q[4 * c + 2], rRw[4 * c + 2]);
                        o.w = mul_bf16x2(q[4 * c + 3], rRw[4 * c + 3]);
                        st_shared_v4(sQp + sw128_offset<TILE>(tid, c), o.x, o.y, o.z, o.w);
                    }
                }
                fence_async_smem();
                tc_fence_before();
                __syncthreads();
                if (warp == 0) {   // converged warp, MMAs and commit predicated on its elected lane
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < DP / 16; ++kk) {
                        const uint32_t off = ((kk >> 2) * (TILE * 128) + (kk & 3) * 32) / 16;
                        umma_ss_pred(tmem_base, dQp + off, dC + off, idesc_x, kk > 0, issuer);
                    }
                    umma_commit_pred(bar, issuer);
                    if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
                }
                phase ^= 1;
                __syncthreads();
                tc_fence_after();
                if (*sFail) { failed = true; break; }

                // --- per-row softmax over the tile's visible columns ------------------------------
                float m_row = -INFINITY, l_row = 0.f;
                if (SC) {
                    // weights of the scatter form: one pass, no maximum
                    uint32_t x[32];
                    const float c2x2 = 2.f * c2;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld32(tX + c * 32, x);
                        tmem_wait_ld();
                        const uint32_t vw = my_vis ? ((c == 0 ? vc0 : c == 1 ? vc1 : c == 2 ? vc2 : vc3) &
                                                      (c == 0 ? pw0 : c == 1 ? pw1 : c == 2 ? pw2 : pw3)) : 0u;
                        const float* lc = sColL + c * 32;
                        uint32_t pk[16];
#pragma unroll
                        for (int t = 0; t < 32; t += 2) {
                            float e0 = fast_exp2(fmaf(__uint_as_float(x[t]), c2x2, -(lse_row + lc[t])));
                            float e1 = fast_exp2(fmaf(__uint_as_float(x[t + 1]), c2x2, -(lse_row + lc[t + 1])));
                            if (!((vw >> t) & 1u)) e0 = 0.f;
                            if (!((vw >> (t + 1)) & 1u)) e1 = 0.f;
                            pk[t >> 1] = pack_bf16x2(e0, e1);
                        }
                        tmem_st16(tX + c * 16, pk);
                    }
                    m_row = 0.f;
                } else {
                    uint32_t x[32];
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld32(tX + c * 32, x);
                        tmem_wait_ld();
                        const uint32_t vw = my_vis ? (c == 0 ? vc0 : c == 1 ? vc1 : c == 2 ? vc2 : vc3) : 0u;
                        // four independent running maxima instead of one chain of 32 dependent operations
                        float m0 = m_row, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
                        if (vw == 0xFFFFFFFFu) {
#pragma unroll
                            for (int t = 0; t < 32; t += 8) {
                                m0 = fmaxf(m0, fmaxf(__uint_as_float(x[t]), __uint_as_float(x[t + 1])));
                                m1 = fmaxf(m1, fmaxf(__uint_as_float(x[t + 2]), __uint_as_float(x[t + 3])));
                                m2 = fmaxf(m2, fmaxf(__uint_as_float(x[t + 4]), __uint_as_float(x[t + 5])));
                                m3 = fmaxf(m3, fmaxf(__uint_as_float(x[t + 6]), __uint_as_float(x[t + 7])));
                            }
                        } else {
#pragma unroll
                            for (int t = 0; t < 32; t += 4) {
                                if ((vw >> t) & 1u) m0 = fmaxf(m0, __uint_as_float(x[t]));
                                if ((vw >> (t + 1)) & 1u) m1 = fmaxf(m1, __uint_as_float(x[t + 1]));
                                if ((vw >> (t + 2)) & 1u) m2 = fmaxf(m2, __uint_as_float(x[t + 2]));
                                if ((vw >> (t + 3)) & 1u) m3 = fmaxf(m3, __uint_as_float(x[t + 3]));
                            }
                        }
                        m_row = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                    }
                    const bool live = m_row > -INFINITY;
                    const float mc = (live ? m_row : 0.f) * c2;
                    // packed FP32 arithmetic: one instruction for the exponents of two columns, one for their sums
                    const uint64_t c2p = pair_f32(c2, c2), mcp = pair_f32(-mc, -mc);
                    uint64_t ls0 = pair_f32(0.f, 0.f), ls1 = ls0;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld32(tX + c * 32, x);
                        tmem_wait_ld();
                        const uint32_t vw = live ? (c == 0 ? vc0 : c == 1 ? vc1 : c == 2 ? vc2 : vc3) : 0u;
                        uint32_t pk[16];
#pragma unroll
                        for (int t = 0; t < 32; t += 2) {
                            float a0, a1;
                            unpair_f32(fma_f32x2(pair_b32(x[t], x[t + 1]), c2p, mcp), a0, a1);
                            float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
                            if (!all_cols || !live) {
                                if (!((vw >> t) & 1u)) e0 = 0.f;
                                if (!((vw >> (t + 1)) & 1u)) e1 = 0.f;
                            }
                            if (t & 2) ls1 = add_f32x2(ls1, pair_f32(e0, e1));
                            else ls0 = add_f32x2(ls0, pair_f32(e0, e1));
                            pk[t >> 1] = pack_bf16x2(e0, e1);
                        }
                        tmem_st16(tX + c * 16, pk);
                    }
                    {
                        float s0, s1;
                        unpair_f32(add_f32x2(ls0, ls1), s0, s1);
                        l_row = s0 + s1;
                    }
                }
                tmem_wait_st();
                float m_w = m_row;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) m_w = fmaxf(m_w, __shfl_xor_sync(0xFFFFFFFFu, m_w, o));
                if (lane == 0) sMpart[warp] = m_w;
                tc_fence_before();
                __syncthreads();
                if (warp == 0) {   // converged warp, MMAs and commit predicated on its elected lane
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < TILE / 16; ++kk)
                        umma_ts_pred(tmem_base + 128, tmem_base + kk * 8, dVcM + kk * (2048 / 16), idesc_u, kk > 0, issuer);
                    umma_commit_pred(bar, issuer);
                    if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
                }
                phase ^= 1;
                const float Mt = fmaxf(fmaxf(sMpart[0], sMpart[1]), fmaxf(sMpart[2], sMpart[3]));
                const float w_row = SC ? 1.f : (m_row > -INFINITY) ? fast_exp2((m_row - Mt) * c2) : 0.f;
                __syncthreads();
                tc_fence_after();
                if (*sFail) { failed = true; break; }

                // --- collapse and merge into the anchor's running state ---------------------------
                {
                    uint32_t u[32], w[16];
                    const uint64_t wp = pair_f32(w_row, w_row);
#pragma unroll
                    for (int c = 0; c < DP / 32; ++c) {
                        tmem_ld32(tU + c * 32, u);
                        tmem_wait_ld();
                        // the row's weight in FP32, then BF16 pairs: the product with the packed Vr words and the lane
                        // sum work on pairs (as in the windowed kernels)
#pragma unroll
                        for (int t = 0; t < 32; t += 2) {
                            float a0, a1;
                            unpair_f32(mul_f32x2(pair_b32(u[t], u[t + 1]), wp), a0, a1);
                            w[t >> 1] = mul_bf16x2(pack_bf16x2(a0, a1), rVr[c * 16 + (t >> 1)]);
                        }
                        const float s = sgring::warp_transpose_sum_words(w, lane);
                        sRed[warp * (DP + 4) + c * 32 + lane] = s;
                    }
                    float wl = w_row * l_row;
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) wl += __shfl_xor_sync(0xFFFFFFFFu, wl, o);
                    if (lane == 0) sRed[warp * (DP + 4) + DP] = wl;
                }
                tc_fence_before();
                __syncthreads();
                if (SC) {
                    float* st = sState + (a - a0) * (DP + 4);
                    if (tid < DP)
                        st[tid] += sRed[tid] + sRed[(DP + 4) + tid] + sRed[2 * (DP + 4) + tid] + sRed[3 * (DP + 4) + tid];
                } else if (Mt > -INFINITY) {
                    float* st = sState + (a - a0) * (DP + 4);
                    const float M_old = st[DP];
                    const float M_new = fmaxf(M_old, Mt);
                    const float f_old = (M_old > -INFINITY) ? fast_exp2((M_old - M_new) * c2) : 0.f;
                    const float f_new = fast_exp2((Mt - M_new) * c2);
                    float add = 0.f;
                    if (tid < DP)
                        add = sRed[tid] + sRed[(DP + 4) + tid] + sRed[2 * (DP + 4) + tid] + sRed[3 * (DP + 4) + tid];
                    const float Lt = sRed[DP] + sRed[(DP + 4) + DP] + sRed[2 * (DP + 4) + DP] + sRed[3 * (DP + 4) + DP];
                    const float L_old = st[DP + 1];
                    __syncthreads();                       // everyone has read the old max and sum
                    if (tid < DP) st[tid] = st[tid] * f_old + add * f_new;
                    if (tid == 0) { st[DP] = M_new; st[DP + 1] = L_old * f_old + Lt * f_new; }
                }
                __syncthreads();
            }
        }
    }
    if (!failed) {
        for (int a = a0; a < a1; ++a) {
            const float* st = sState + (a - a0) * (DP + 4);
            const float M = st[DP], Ls = st[DP + 1];
            const size_t row = bh + a;
            if (SC) {
                if (tid < D) p.Y[row * D + tid] = __float2bfloat16(st[tid]);
                continue;
            }
            const bool live = M > -INFINITY && Ls > 0.f;
            if (tid < D) p.Y[row * D + tid] = __float2bfloat16(live ? st[tid] / Ls : 0.f);
            if (tid == 0) { p.m[row] = live ? M * p.scale : NEG_INF_F; p.l[row] = live ? Ls : 0.f; }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 4);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace agdense
