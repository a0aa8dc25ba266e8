// Dense anchored gather, backward, for sm_100a.
//
// Gradients of the operator of ag_dense_fwd.cuh for one key side per launch.  With
// the side whose gradients are produced called "own" (Kb, Vb) and the other side
// (Ka, Va), anchor rows A_a, cotangent dY_a, delta_a = dY_a . Y_a and the forward
// statistics (m_a, l_a):
//
//   P^T[k][j]  = exp(scale * sum_d Kb_k[d] A_a[d] Ka_j[d] - LSE_a)       (visible pairs only)
//   gA^T       = P^T o (sum_d Vb_k[d] dY_a[d] Va_j[d] - delta_a)
//   dKb[k] += scale * sum_{a,j} gA^T[k][j] (A_a o Ka_j)       dVb[k] += sum_{a,j} P^T[k][j] (dY_a o Va_j)
//   dA[a]  += scale * sum_k Kb_k o (sum_j gA^T[k][j] Ka_j)    (on request)
//
// i.e. the algebra of the reference's anchored backward kernel
// (cuda/backward.cu:415-934) with one softmax kept; the three-gather backward is the
// sum of three such gathers with permuted roles, each run as two of these launches
// (own = cols with the anchor gradient, then own = rows).
//
// Schedule: a CTA owns one 128-key tile of the own side for one (batch, head).  Its
// two FP32 accumulators (dKb, dVb tile) stay in tensor memory for the whole kernel
// while it loops over the other side's tiles and, inside, over every anchor; each
// (anchor, tile pair) runs the six-MMA step of the windowed backward
// (sg_ring_bwd.cuh) with the ring replaced by explicit tiles.  The accumulators are
// added to the FP32 outputs once, at the end, by their only owner, so the result is
// deterministic.  The anchor gradient is summed over the other-side tiles by the
// CTA itself (read-modify-write of its own partial plane) and over own-side tiles
// by the caller, which passes one partial plane per own-side tile.
#pragma once

#include "ag_dense_fwd.cuh"

namespace agdense {

constexpr int BWD_THREADS = 256;

struct BwdParams {
    const __nv_bfloat16* A;          // anchor rows         [B,H,NA,D]  (dY, Y, m, l likewise)
    const __nv_bfloat16* dY;         // cotangent of the gather's output
    const __nv_bfloat16* Y;          // the gather's output
    const float* m;                  // [B,H,N] statistics of the gather (per anchor)
    const float* l;
    const __nv_bfloat16* Ka;         // other side          [B,H,N_oth,D]
    const __nv_bfloat16* Va;
    const __nv_bfloat16* Kb;         // own side            [B,H,N_own,D]
    const __nv_bfloat16* Vb;
    const uint8_t* mask;             // [B,N,N] or null (then NA = N_own = N_oth = N)
    float* dKb;                      // [B,H,N_own,D] FP32, this kernel adds into it
    float* dVb;
    float* dA_part;                  // [own tiles][B,H,NA,D] FP32 partial planes, zero-filled by the caller
    // Anchor chunks: with few (tile, batch, head) triples the anchors are split over a_chunks CTAs per
    // triple (grid.x = n_tiles * a_chunks).  Chunk 0 adds into dKb / dVb; chunk 1 adds into its own
    // zero-filled planes, which the caller adds afterwards, so the order of the sums stays fixed.
    int a_chunks;                    // 1 or 2
    float* dKb1;
    float* dVb1;
    // Lengths of the anchor, own-side and other-side axes and how many leading entries of each are real (0 or > length:
    // all); a_valid only matters to the scatter forms.
    int B, H, NA, N_own, N_oth, D, a_valid, own_valid, oth_valid;
    float scale;
    int* status;
    // Scatter forms (SC = 1, 2): statistics of the softmaxes anchored at the own and at the other index, and
    // (SC = 2) the correction sums C[x] = V2[x] . dV2[x] of the two indices           [B,H,N] each
    const float* m_own; const float* l_own;
    const float* m_oth; const float* l_oth;
    const float* C_own; const float* C_oth;
};

template <int DP, bool WITH_DA>
struct BwdSmem {
    static constexpr int TILE_BYTES = TILE * DP * 2;
    static constexpr int OFF_KB = 0;
    static constexpr int OFF_VB = TILE_BYTES;
    static constexpr int OFF_QP = 2 * TILE_BYTES;
    static constexpr int OFF_G = 3 * TILE_BYTES;
    static constexpr int OFF_KA = 4 * TILE_BYTES;                       // only WITH_DA
    static constexpr int OFF_RED = (WITH_DA ? 5 : 4) * TILE_BYTES;      // 4 x DP floats
    static constexpr int OFF_VIS = OFF_RED + 4 * DP * 4;                // 4 own words + 4 other words
    static constexpr int OFF_MISC = OFF_VIS + 32;
    static constexpr int OFF_COL = OFF_MISC + 16;                       // scatter forms: 2 x 128 other-side constants
    static constexpr int BYTES = OFF_COL + 2 * TILE * 4;
    static constexpr int ALLOC = BYTES + 1024;
};

// SC = 1 and SC = 2 are the two backward passes of one scatter output of the three-gather operator
// (cuda/backward.cu:175-316, 949-1613) in the same schedule.  With the output index as the anchor a, the
// cotangent g[a] in the place of dY, the second value tensors in the place of Va / Vb, and
//   Po = exp(x - LSE_own[k]),  Pt = exp(x - LSE_oth[j]),  W = Po Pt,  c = sum_d g[a,d] Vb[k,d] Va[j,d]:
//   SC = 1:  dVb[k] += sum_{a,j} W (g[a] o Va[j])                      (P^T := W, gA^T := 0)
//   SC = 2:  dx = 2 W c - Po C_own[k] - Pt C_oth[j];  dKb[k] += scale sum_{a,j} dx (A_a o Ka_j) and, on
//            request, dA[a] += scale sum_k Kb_k o (sum_j dx Ka_j)      (P^T := 0, gA^T := dx)
// Po is live iff anchor k sees a and j (mask[k][a], mask[k][j]), Pt iff anchor j sees a and k; W needs both.
// The MMA sequence is the gather's, so one of the two accumulations adds zeros in each pass.
template <int DP, bool WITH_DA, int SC = 0>
__global__ void __launch_bounds__(BWD_THREADS, 1) ag_dense_bwd_kernel(const BwdParams p) {
    using L = BwdSmem<DP, WITH_DA>;
    constexpr int HD = DP / 2, HCH = HD / 8, HW = HD / 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t C_XT = 0, C_DP = 128, C_AK = 256, C_AV = 384, C_W0 = 64, C_W1 = 192;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKb = smem + L::OFF_KB;
    uint8_t* sVb = smem + L::OFF_VB;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sG = smem + L::OFF_G;
    uint8_t* sKa = smem + L::OFF_KA;
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + L::OFF_VIS);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC + 8);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 12);
    float* sColL = reinterpret_cast<float*>(smem + L::OFF_COL);          // LSE of the other-side anchors (log2 units)
    float* sColC = sColL + TILE;                                         // their correction sums

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t issuer = elect_one();     // one lane per warp; warp 0 predicates its MMAs on it
    const int slot = tid & (TILE - 1);
    const int half = tid >> 7;
    const int b = blockIdx.z, h = blockIdx.y;
    const int N = p.NA, D = p.D;                 // N: the mask's side (a mask needs equal lengths)
    const int n_own = (p.own_valid > 0 && p.own_valid < p.N_own) ? p.own_valid : p.N_own;
    const int n_oth = (p.oth_valid > 0 && p.oth_valid < p.N_oth) ? p.oth_valid : p.N_oth;
    const int n_anch = (p.a_valid > 0 && p.a_valid < p.NA) ? p.a_valid : p.NA;
    const int own_tiles = (n_own + TILE - 1) / TILE, oth_tiles = (n_oth + TILE - 1) / TILE;
    const int kb = blockIdx.x % own_tiles, chunk = blockIdx.x / own_tiles;
    const int n_anchors = SC ? n_anch : p.NA;         // padded anchors take no part in a scatter sum
    const int a_begin = static_cast<int>((static_cast<long long>(n_anchors) * chunk) / p.a_chunks);
    const int a_end = static_cast<int>((static_cast<long long>(n_anchors) * (chunk + 1)) / p.a_chunks);

    if (warp == 0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        *sFail = 0;
    }
    const size_t bh = (static_cast<size_t>(b) * p.H + h) * p.NA;                   // anchor-indexed arrays
    const size_t bh_own = (static_cast<size_t>(b) * p.H + h) * p.N_own, bh_oth = (static_cast<size_t>(b) * p.H + h) * p.N_oth;
    const __nv_bfloat16* gA = p.A + bh * D;
    const __nv_bfloat16* gdY = p.dY + bh * D;
    const __nv_bfloat16* gY = p.Y + bh * D;
    const __nv_bfloat16* gKa = p.Ka + bh_oth * D;
    const __nv_bfloat16* gVa = p.Va + bh_oth * D;
    const __nv_bfloat16* gKb = p.Kb + bh_own * D;
    const __nv_bfloat16* gVb = p.Vb + bh_own * D;
    const uint8_t* mask_b = p.mask ? p.mask + static_cast<size_t>(b) * N * N : nullptr;
    const int own_key = kb * TILE + slot;

    // Own tile into shared memory (this thread: half a row of each tensor), zero-padded.
    auto store_half_row = [&](uint8_t* dst, const __nv_bfloat16* src, int idx) {
#pragma unroll
        for (int c = 0; c < HCH; ++c) {
            const int cc = half * HCH + c;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (idx < n_own && cc * 8 < D) v = __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(idx) * D) + cc);
            *reinterpret_cast<uint4*>(dst + sw128_offset<TILE>(slot, cc)) = v;
        }
    };
    store_half_row(sKb, gKb, own_key);
    store_half_row(sVb, gVb, own_key);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tl = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    {
        uint32_t z[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) z[t] = 0;
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) tmem_st32(tl + (half ? C_AV : C_AK) + c * 32, z);
        tmem_wait_st();
    }
    const uint32_t idesc_s = make_idesc_bf16(TILE, TILE, 0, 0);
    const uint32_t idesc_acc = make_idesc_bf16(TILE, DP, 0, 1);
    const uint32_t idesc_w = make_idesc_bf16(TILE, 64, 0, 1);
    const uint64_t dKb = make_smem_desc(smem_u32(sKb), 16, 1024, SWIZZLE_128B);
    const uint64_t dVb = make_smem_desc(smem_u32(sVb), 16, 1024, SWIZZLE_128B);
    const uint64_t dQpK = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);
    const uint64_t dGK = make_smem_desc(smem_u32(sG), 16, 1024, SWIZZLE_128B);
    const uint64_t dQpM = make_smem_desc(smem_u32(sQp), TILE * 128, 1024, SWIZZLE_128B);
    const uint64_t dGM = make_smem_desc(smem_u32(sG), TILE * 128, 1024, SWIZZLE_128B);
    const uint64_t dKaM = make_smem_desc(smem_u32(sKa), TILE * 128, 1024, SWIZZLE_128B);
    const float c2 = p.scale * LOG2E;
    uint32_t phase = 0;
    bool failed = false;
    float* gPart = WITH_DA ? p.dA_part + (static_cast<size_t>(kb) * p.B * p.H * p.NA + bh) * D : nullptr;
    // scatter forms: constants of this thread's own key; a dead or padded anchor gets an LSE that makes its
    // softmax vanish
    float lse_own = 1e30f, c_own = 0.f;
    if (SC && own_key < n_own) {
        const float lo = __ldg(p.l_own + bh_own + own_key);
        if (lo > 0.f) lse_own = __ldg(p.m_own + bh_own + own_key) * LOG2E + __log2f(lo);
        if (SC == 2) c_own = __ldg(p.C_own + bh_own + own_key);
    }

    for (int jb = 0; jb < oth_tiles && !failed; ++jb) {
        // other-side tile: this thread's half row of Ka and Va in registers (Ka also in smem for W)
        uint32_t rKa[HW], rVa[HW];
        const int oth_key = jb * TILE + slot;
#pragma unroll
        for (int c = 0; c < HCH; ++c) {
            const int cc = half * HCH + c;
            uint4 a = make_uint4(0, 0, 0, 0), v = a;
            if (oth_key < n_oth && cc * 8 < D) {
                a = __ldg(reinterpret_cast<const uint4*>(gKa + static_cast<size_t>(oth_key) * D) + cc);
                v = __ldg(reinterpret_cast<const uint4*>(gVa + static_cast<size_t>(oth_key) * D) + cc);
            }
            rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
            rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
            if (WITH_DA) *reinterpret_cast<uint4*>(sKa + sw128_offset<TILE>(slot, cc)) = a;
        }
        // scatter forms: constants of the other-side keys of this tile, and for this thread's two 32-column
        // chunks (c = 2 rd + half) the pairs in which anchor k sees j (pbo) and anchor j sees k (pbt)
        uint32_t pbo0 = 0, pbo1 = 0, pbt0 = 0, pbt1 = 0;
        if (SC) {
            if (half == 0) {
                float lt = 1e30f, ct = 0.f;
                if (oth_key < n_oth) {
                    const float l = __ldg(p.l_oth + bh_oth + oth_key);
                    if (l > 0.f) lt = __ldg(p.m_oth + bh_oth + oth_key) * LOG2E + __log2f(l);
                    if (SC == 2) ct = __ldg(p.C_oth + bh_oth + oth_key);
                }
                sColL[slot] = lt;
                sColC[slot] = ct;
            }
            if (own_key < n_own) {
#pragma unroll 1
                for (int rd = 0; rd < 2; ++rd) {
                    uint32_t wo = 0, wt = 0;
                    for (int t = 0; t < 32; ++t) {
                        const int j = jb * TILE + (2 * rd + half) * 32 + t;
                        if (j >= n_oth) break;
                        const bool so = !mask_b || mask_b[static_cast<size_t>(own_key) * N + j] != 0;
                        const bool st = !mask_b || mask_b[static_cast<size_t>(j) * N + own_key] != 0;
                        wo |= static_cast<uint32_t>(so) << t;
                        wt |= static_cast<uint32_t>(st) << t;
                    }
                    if (rd == 0) { pbo0 = wo; pbt0 = wt; } else { pbo1 = wo; pbt1 = wt; }
                }
            }
        }
        fence_async_smem();

        for (int a = a_begin; a < a_end && !failed; ++a) {
            // visibility from anchor a: own-side keys of this tile, other-side keys of tile jb
            {
                bool vo = own_key < n_own, vt = oth_key < n_oth;
                if (mask_b && SC) {
                    // the anchors of the two softmaxes are the own and the other key: each must see a
                    if (vo) vo = mask_b[static_cast<size_t>(own_key) * N + a] != 0;
                    if (vt) vt = mask_b[static_cast<size_t>(oth_key) * N + a] != 0;
                } else if (mask_b) {
                    const uint8_t* mrow = mask_b + static_cast<size_t>(a) * N;
                    if (vo) vo = mrow[own_key] != 0;
                    if (vt) vt = mrow[oth_key] != 0;
                }
                const uint32_t wo = __ballot_sync(0xFFFFFFFFu, vo), wt = __ballot_sync(0xFFFFFFFFu, vt);
                if (lane == 0 && warp < 4) { sVis[warp] = wo; sVis[4 + warp] = wt; }
            }
            const float m_a = SC ? 0.f : __ldg(p.m + bh + a), l_a = SC ? 1.f : __ldg(p.l + bh + a);
            tc_fence_before();
            __syncthreads();
            tc_fence_after();
            const uint32_t vo_any = sVis[0] | sVis[1] | sVis[2] | sVis[3];
            const uint32_t vt0 = sVis[4], vt1 = sVis[5], vt2 = sVis[6], vt3 = sVis[7];
            const bool my_vis = (sVis[warp & 3] >> lane) & 1u;
            if (vo_any == 0 || (vt0 | vt1 | vt2 | vt3) == 0 || !(l_a > 0.f)) {
                __syncthreads();
                continue;
            }
            // delta = dY_a . Y_a (same value in every warp), log-sum-exp in log2 units
            float delta = 0.f;
            if (!SC) {
                for (int t = lane; t < D; t += 32)
                    delta += __bfloat162float(gdY[static_cast<size_t>(a) * D + t]) * __bfloat162float(gY[static_cast<size_t>(a) * D + t]);
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) delta += __shfl_xor_sync(0xFFFFFFFFu, delta, o);
            }
            const float lse2 = m_a * LOG2E + __log2f(l_a);
            const uint64_t c2p = pair_f32(c2, c2), lsep = pair_f32(-lse2, -lse2), dltp = pair_f32(-delta, -delta);

            // --- Hadamard tiles (this thread: half a row) -----------------------------------------
#pragma unroll
            for (int c = 0; c < HCH; ++c) {
                const int cc = half * HCH + c;
                uint4 q = make_uint4(0, 0, 0, 0), y = q;
                if (cc * 8 < D) {
                    q = __ldg(reinterpret_cast<const uint4*>(gA + static_cast<size_t>(a) * D) + cc);
                    y = __ldg(reinterpret_cast<const uint4*>(gdY + static_cast<size_t>(a) * D) + cc);
                }
                uint4 o, gq;
                o.x = mul_bf16x2(q.x, rKa[4 * c]);      gq.x = mul_bf16x2(y.x, rVa[4 * c]);
                o.y = mul_bf16x2(q.y, rKa[4 * c + 1]);  gq.y = mul_bf16x2(y.y, rVa[4 * c + 1]);
                o.z = mul_bf16x2(q.z, rKa[4 * c + 2]);  gq.z = mul_bf16x2(y.z, rVa[4 * c + 2]);
                o.w = mul_bf16x2(q.w, rKa[4 * c + 3]);  gq.w = mul_bf16x2(y.w, rVa[4 * c + 3]);
                st_shared_v4(sQp + sw128_offset<TILE>(slot, cc), o.x, o.y, o.z, o.w);
                st_shared_v4(sG + sw128_offset<TILE>(slot, cc), gq.x, gq.y, gq.z, gq.w);
            }
            fence_async_smem();
            tc_fence_before();
            __syncthreads();
            if (warp == 0) {   // converged warp, MMAs and commit predicated on its elected lane
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < DP / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * (TILE * 128) + (kk & 3) * 32) / 16;
                    umma_ss_pred(tmem_base + C_XT, dKb + off, dQpK + off, idesc_s, kk > 0, issuer);
                }
#pragma unroll
                for (int kk = 0; kk < DP / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * (TILE * 128) + (kk & 3) * 32) / 16;
                    umma_ss_pred(tmem_base + C_DP, dVb + off, dGK + off, idesc_s, kk > 0, issuer);
                }
                umma_commit_pred(bar, issuer);
                if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
            }
            phase ^= 1;
            __syncthreads();
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            // --- P^T and gA^T; round rd covers chunks 2rd (half 0) and 2rd+1 (half 1) ------------
            const int n_own = __popc(sVis[0]) + __popc(sVis[1]) + __popc(sVis[2]) + __popc(sVis[3]);
            const int n_oth = __popc(vt0) + __popc(vt1) + __popc(vt2) + __popc(vt3);
            (void)n_own; (void)n_oth;
#pragma unroll 1
            for (int rd = 0; rd < 2; ++rd) {
                const int c = 2 * rd + half;
                uint32_t x[32], dp[32], pk[16], gk[16];
                tmem_ld32(tl + C_XT + c * 32, x);
                tmem_ld32(tl + C_DP + c * 32, dp);
                tmem_wait_ld();
                const uint32_t vtw = rd == 0 ? (half ? vt1 : vt0) : (half ? vt3 : vt2);
                const uint32_t cw = my_vis ? vtw : 0u;
                if (SC) {
                    // supports: Po needs anchor k to see a (my_vis) and j (pbo); Pt needs anchor j to see a (vtw) and k (pbt)
                    const uint32_t so = my_vis ? (rd == 0 ? pbo0 : pbo1) : 0u;
                    const uint32_t st = vtw & (rd == 0 ? pbt0 : pbt1);
                    const float* lt = sColL + c * 32;
                    const float* ct = sColC + c * 32;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        const float xs0 = __uint_as_float(x[t]) * c2, xs1 = __uint_as_float(x[t + 1]) * c2;
                        const float po0 = ((so >> t) & 1u) ? fast_exp2(xs0 - lse_own) : 0.f;
                        const float po1 = ((so >> (t + 1)) & 1u) ? fast_exp2(xs1 - lse_own) : 0.f;
                        const float pt0 = ((st >> t) & 1u) ? fast_exp2(xs0 - lt[t]) : 0.f;
                        const float pt1 = ((st >> (t + 1)) & 1u) ? fast_exp2(xs1 - lt[t + 1]) : 0.f;
                        const float w0 = po0 * pt0, w1 = po1 * pt1;
                        if (SC == 1) {
                            pk[t >> 1] = pack_bf16x2(w0, w1);
                            gk[t >> 1] = 0u;
                        } else {
                            const float d0 = 2.f * w0 * __uint_as_float(dp[t]) - po0 * c_own - pt0 * ct[t];
                            const float d1 = 2.f * w1 * __uint_as_float(dp[t + 1]) - po1 * c_own - pt1 * ct[t + 1];
                            pk[t >> 1] = 0u;
                            gk[t >> 1] = pack_bf16x2(d0, d1);
                        }
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        // packed FP32 arithmetic: two columns an instruction
                        float a0, a1;
                        unpair_f32(fma_f32x2(pair_b32(x[t], x[t + 1]), c2p, lsep), a0, a1);
                        float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                        if (!((cw >> t) & 1u)) p0 = 0.f;
                        if (!((cw >> (t + 1)) & 1u)) p1 = 0.f;
                        float g0, g1;
                        unpair_f32(mul_f32x2(pair_f32(p0, p1), add_f32x2(pair_b32(dp[t], dp[t + 1]), dltp)), g0, g1);
                        pk[t >> 1] = pack_bf16x2(p0, p1);
                        gk[t >> 1] = pack_bf16x2(g0, g1);
                    }
                }
                if (rd == 0) {
                    tc_fence_before();
                    __syncthreads();
                    tc_fence_after();
                }
                tmem_st16(tl + C_XT + c * 16, pk);
                tmem_st16(tl + C_DP + c * 16, gk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncthreads();
            if (warp == 0) {   // converged warp, MMAs and commit predicated on its elected lane
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < TILE / 16; ++kk)
                    umma_ts_pred(tmem_base + C_AK, tmem_base + C_DP + kk * 8, dQpM + kk * (2048 / 16), idesc_acc, 1, issuer);
#pragma unroll
                for (int kk = 0; kk < TILE / 16; ++kk)
                    umma_ts_pred(tmem_base + C_AV, tmem_base + C_XT + kk * 8, dGM + kk * (2048 / 16), idesc_acc, 1, issuer);
                if (WITH_DA) {
#pragma unroll
                    for (int dh = 0; dh < DP / 64; ++dh)
#pragma unroll
                        for (int kk = 0; kk < TILE / 16; ++kk)
                            umma_ts_pred(tmem_base + (dh ? C_W1 : C_W0), tmem_base + C_DP + kk * 8,
                                         dKaM + (dh * (TILE * 128) + kk * 2048) / 16, idesc_w, kk > 0, issuer);
                }
                umma_commit_pred(bar, issuer);
                if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
            }
            phase ^= 1;
            __syncthreads();
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            if (WITH_DA) {
                const uint32_t wcol = (DP == 128) ? (half ? C_W1 : C_W0) : (C_W0 + half * 32);
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t u[32], w[16];
                    tmem_ld32(tl + wcol + c * 32, u);
                    tmem_wait_ld();
                    // W rounded to BF16 pairs and multiplied by the packed Kb words as they are; the lane sum works on
                    // pairs (as in the windowed kernels)
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 kbv =
                            *reinterpret_cast<const uint4*>(sKb + sw128_offset<TILE>(slot, half * HCH + c * 4 + q));
                        const uint32_t w4[4] = {kbv.x, kbv.y, kbv.z, kbv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[q * 4 + e] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[q * 8 + 2 * e]),
                                                                  __uint_as_float(u[q * 8 + 2 * e + 1])), w4[e]);
                    }
                    const float s = sgring::warp_transpose_sum_words(w, lane);
                    sRed[(warp & 3) * DP + half * HD + c * 32 + lane] = s;
                }
                tc_fence_before();
                __syncthreads();
                if (tid < D) {
                    float* dst = gPart + static_cast<size_t>(a) * D + tid;
                    *dst += p.scale * (sRed[tid] + sRed[DP + tid] + sRed[2 * DP + tid] + sRed[3 * DP + tid]);
                }
            }
            __syncthreads();
        }
    }
    // Add the tile's accumulators into the FP32 outputs (this CTA is the only writer of these rows).
    // (scatter forms: only the accumulator that received something is added, dVb in pass 1, dKb in pass 2)
    if (!failed && (SC == 0 || (SC == 1) == (half == 1))) {
        float* dst_base = chunk == 0 ? (half ? p.dVb : p.dKb) : (half ? p.dVb1 : p.dKb1);
        const float mul = half ? 1.0f : p.scale;
        uint32_t acc[32];
#pragma unroll 1
        for (int c = 0; c < DP / 32; ++c) {
            tmem_ld32(tl + (half ? C_AV : C_AK) + c * 32, acc);
            tmem_wait_ld();
            if (own_key < n_own) {
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    const int d = c * 32 + t;
                    if (d < D) dst_base[(bh_own + own_key) * D + d] += mul * __uint_as_float(acc[t]);
                }
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 5);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// out_bf16[i] = bf16(a[i] (+ b[i] + c[i] ...)): sums up to `n_src` FP32 planes laid out
// plane-major (stride `plane` elements) and rounds once.
__global__ void ag_sum_planes_to_bf16(const float* src, int n_src, size_t plane, __nv_bfloat16* out, size_t n) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < n_src; ++k) s += src[k * plane + i];
        out[i] = __float2bfloat16(s);
    }
}

// acc[i] += sum_k src[k][i]  (FP32), for folding anchor-gradient partial planes into a total.
__global__ void ag_add_planes(const float* src, int n_src, size_t plane, float* acc, size_t n) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float s = acc[i];
        for (int k = 0; k < n_src; ++k) s += src[k * plane + i];
        acc[i] = s;
    }
}


// row . row over D for two [n, D] tensors (bf16 x fp32): C[n] = sum_d V2[n,d] * dV2[n,d]
__global__ void rowdot_kernel(const __nv_bfloat16* v2, const float* dv2, float* out, size_t rows, int D) {
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) / 32;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += __bfloat162float(v2[warp * D + d]) * dv2[warp * D + d];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if (lane == 0) out[warp] = s;
}

}  // namespace agdense
