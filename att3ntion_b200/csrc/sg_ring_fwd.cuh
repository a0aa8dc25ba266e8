// Windowed single-gather forward for sm_100a ("ring" schedule).
//
//   Y[i] = sum_{j,k} softmax_{(j,k)}( scale * sum_d Q_i[d] R_j[d] S_k[d] ) Vr[j] o Vs[k]
//
// with both keys restricted to the causal window (i - w, i], w <= 128.  This is
// the operator of the reference's Y_gather_tc / shared-KV forward kernels
// (cuda/forward.cu:108-477; cuda/shared_kv/shared_retained_fwd.cuh) re-derived
// for tcgen05:
//
//  * A CTA owns a contiguous block of queries of one (batch, KV head) and walks
//    them in order, looping over the query heads that share the KV head.  The
//    128 most recent keys live in a ring: key k sits in slot k mod 128 of the
//    S and Vs shared-memory tiles (and of the per-thread R / Vr registers), so
//    sliding the window by one query rewrites exactly one row and the MMA
//    operands never move.  Contractions over the ring are order independent,
//    which is what makes the rotated order legal.
//  * Per (query, head):  X = (Q_i o R) S^T  is one 128x128xD tcgen05.mma with
//    the Hadamard tile built in shared memory; thread j owns row j of X in
//    tensor memory, takes its row maximum and writes P = exp2(.) back to tensor
//    memory as BF16 over the consumed score columns; U = P Vs is the second MMA
//    with A read from tensor memory and the Vs ring as an MN-major B operand;
//    the epilogue collapses  sum_j w_j Vr_j o U_j  with warp shuffles, where
//    w_j = exp(m_j - M) merges the per-row softmaxes into the joint one.
//  * The score scale is folded into the exp2 argument, so the only BF16
//    rounding before the score MMA is the product Q_i[d] * R_j[d] itself.
#pragma once

#include "sm100_ptx.cuh"

namespace sgring {

using namespace sm100;

constexpr int RING = 128;          // keys resident per CTA = maximum window
constexpr int NTHREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_INF_F = -1e30f;   // statistics value of a query with no visible pair

struct FwdParams {
    const __nv_bfloat16* Q;        // [B,Hq,N,D]
    const __nv_bfloat16* R;        // [B,Hkv,N,D]
    const __nv_bfloat16* S;
    const __nv_bfloat16* Vr;
    const __nv_bfloat16* Vs;
    const uint8_t* mask;           // [B,N,N] or null
    __nv_bfloat16* Y;              // [B,Hq,N,D]
    float* m;                      // [B,Hq,N]
    float* l;
    int B, Hq, Hkv, N, window, q_begin, block_len;
    float scale;
    int* status;                   // device status word (bounded-wait failures)
};

template <int D>
struct FwdSmem {
    static constexpr int TILE = RING * D * 2;           // bytes of one [128][D] BF16 tile
    static constexpr int OFF_S = 0;
    static constexpr int OFF_VS = TILE;
    static constexpr int OFF_QP = 2 * TILE;
    static constexpr int OFF_QSTAGE = 3 * TILE;         // 2 x D bf16
    static constexpr int OFF_RED = OFF_QSTAGE + 2 * D * 2;   // 4 x (D+1) floats
    static constexpr int OFF_MPART = OFF_RED + 4 * (D + 4) * 4;
    static constexpr int OFF_VIS = OFF_MPART + 16;      // 4 words
    static constexpr int OFF_MISC = OFF_VIS + 16;       // mbarrier (8) + tmem slot (4) + fail (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;          // slack for manual 1024-byte alignment
};

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

template <int D>
__global__ void __launch_bounds__(NTHREADS, 2) sg_ring_fwd_kernel(const FwdParams p) {
    using L = FwdSmem<D>;
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int DW = D / 2;            // packed bf16x2 words per row
    constexpr uint32_t TMEM_COLS = 256;  // X/P [0,128), U [128,128+D)

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sS = smem + L::OFF_S;
    uint8_t* sVs = smem + L::OFF_VS;
    uint8_t* sQp = smem + L::OFF_QP;
    __nv_bfloat16* sQst = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_QSTAGE);
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    float* sMpart = reinterpret_cast<float*>(smem + L::OFF_MPART);
    uint32_t* sVis = reinterpret_cast<uint32_t*>(smem + L::OFF_VIS);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC + 8);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 12);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t issuer = elect_one();     // one lane per warp; warp 0 predicates its MMAs on it
    const int b = blockIdx.z, g = blockIdx.y;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + blockIdx.x * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;

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
    const __nv_bfloat16* gR = p.R + kv_base * D;
    const __nv_bfloat16* gS = p.S + kv_base * D;
    const __nv_bfloat16* gVr = p.Vr + kv_base * D;
    const __nv_bfloat16* gVs = p.Vs + kv_base * D;

    // Ring slot `tid`: R and Vr rows in registers, S and Vs rows in shared memory.
    uint32_t rR[DW], rVr[DW];
    auto load_slot = [&](int key) {
        if (key >= 0) {
            const uint4* r4 = reinterpret_cast<const uint4*>(gR + static_cast<size_t>(key) * D);
            const uint4* vr4 = reinterpret_cast<const uint4*>(gVr + static_cast<size_t>(key) * D);
            const uint4* s4 = reinterpret_cast<const uint4*>(gS + static_cast<size_t>(key) * D);
            const uint4* vs4 = reinterpret_cast<const uint4*>(gVs + static_cast<size_t>(key) * D);
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const uint4 a = __ldg(r4 + c), v = __ldg(vr4 + c);
                rR[4 * c] = a.x; rR[4 * c + 1] = a.y; rR[4 * c + 2] = a.z; rR[4 * c + 3] = a.w;
                rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(tid, c)) = __ldg(s4 + c);
                *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(tid, c)) = __ldg(vs4 + c);
            }
        } else {
            const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                rR[4 * c] = rR[4 * c + 1] = rR[4 * c + 2] = rR[4 * c + 3] = 0;
                rVr[4 * c] = rVr[4 * c + 1] = rVr[4 * c + 2] = rVr[4 * c + 3] = 0;
                *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(tid, c)) = z;
                *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(tid, c)) = z;
            }
        }
    };
    load_slot(ring_key(q0, tid));

    // Q row of the first (query, head) into stage 0.
    auto q_row = [&](int it) {
        const int i = q0 + it / G, h = g * G + it % G;
        return p.Q + ((static_cast<size_t>(b) * p.Hq + h) * p.N + i) * D;
    };
    const int n_iter = (q1 - q0) * G;
    if (tid < CH) reinterpret_cast<uint4*>(sQst)[tid] = __ldg(reinterpret_cast<const uint4*>(q_row(0)) + tid);

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tX = tmem_base + lane_field;          // scores, later P (BF16 pairs) in columns [0,64)
    const uint32_t tU = tmem_base + lane_field + 128;    // P.Vs accumulator

    const uint32_t idesc_x = make_idesc_bf16(RING, RING, 0, 0);
    const uint32_t idesc_u = make_idesc_bf16(RING, D, 0, 1);
    // descriptor bases, built once; a k-step adds a constant to the start-address field
    const uint64_t dQp = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);           // A, K-major
    const uint64_t dS = make_smem_desc(smem_u32(sS), 16, 1024, SWIZZLE_128B);             // B, K-major
    const uint64_t dVsM = make_smem_desc(smem_u32(sVs), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major
    const float c2 = p.scale * LOG2E;
    uint32_t phase = 0;
    bool failed = false;

    int it = 0;
    for (int i = q0; i < q1 && !failed; ++i) {
        // --- slide the window: slot (i mod 128) now holds key i ---------------
        if (i > q0 && tid == (i & (RING - 1))) load_slot(i);
        bool my_vis;
        {
            const int key = ring_key(i, tid);
            my_vis = key >= 0 && key > i - p.window;
            if (my_vis && p.mask) my_vis = p.mask[(static_cast<size_t>(b) * p.N + i) * p.N + key] != 0;
            const uint32_t w = __ballot_sync(0xFFFFFFFFu, my_vis);
            if (lane == 0) sVis[warp] = w;
        }
        __syncthreads();
        const uint32_t vw0 = sVis[0], vw1 = sVis[1], vw2 = sVis[2], vw3 = sVis[3];
        const bool any_vis = (vw0 | vw1 | vw2 | vw3) != 0;
        const bool all_vis = (vw0 & vw1 & vw2 & vw3) == 0xFFFFFFFFu;

        for (int hh = 0; hh < G && !failed; ++hh, ++it) {
            const int h = g * G + hh;
            const size_t row = (static_cast<size_t>(b) * p.Hq + h) * p.N + i;
            // prefetch the next (query, head)'s Q row into the other stage
            if (tid < CH && it + 1 < n_iter) {
                const uint32_t dst = smem_u32(sQst + ((it + 1) & 1) * D) + tid * 16;
                const void* src = reinterpret_cast<const uint4*>(q_row(it + 1)) + tid;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            if (!any_vis) {
                // No visible pair: Y = 0, m = NEG_INF, l = 0 (cuda/common.cuh:24).
                if (tid < D) p.Y[row * D + tid] = __float2bfloat16(0.f);
                if (tid == 0) { p.m[row] = NEG_INF_F; p.l[row] = 0.f; }
                if (tid < CH) asm volatile("cp.async.wait_all;" ::: "memory");
                __syncthreads();
                continue;
            }

            // --- Hadamard tile: Qp[j][d] = bf16(Q_i[d] * R_j[d]) ------------------
            {
                const uint4* q4 = reinterpret_cast<const uint4*>(sQst + (it & 1) * D);
                // Loads of the staged row in batches of eight chunks ahead of the tile stores: the
                // compiler cannot rule out aliasing between the two shared-memory areas and would
                // otherwise serialise load -> multiply -> store per chunk.
#pragma unroll
                for (int c0 = 0; c0 < CH; c0 += 8) {
                    uint4 q[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) q[c] = q4[c0 + c];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4 o;
                        o.x = mul_bf16x2(q[c].x, rR[4 * (c0 + c)]);
                        o.y = mul_bf16x2(q[c].y, rR[4 * (c0 + c) + 1]);
                        o.z = mul_bf16x2(q[c].z, rR[4 * (c0 + c) + 2]);
                        o.w = mul_bf16x2(q[c].w, rR[4 * (c0 + c) + 3]);
                        *reinterpret_cast<uint4*>(sQp + sw128_offset<RING>(tid, c0 + c)) = o;
                    }
                }
            }
            fence_async_smem();
            tc_fence_before();
            __syncthreads();                                           // B1
            if (warp == 0) {
                // the warp stays converged; the MMAs and the commit are predicated on its elected lane
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * (RING * 128) + (kk & 3) * 32) / 16;
                    umma_ss_pred(tmem_base, dQp + off, dS + off, idesc_x, kk > 0, issuer);
                }
                umma_commit_pred(bar, issuer);
                if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
                __syncwarp();
            }
            phase ^= 1;
            __syncthreads();                                           // B2
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            // --- per-row softmax over the 128 ring columns ------------------------
            // tcgen05.ld/st are warp-collective, so every thread runs the same
            // instruction stream; an invisible row is a row whose columns are all
            // masked (rows and columns share one visibility set).
            float m_row = -INFINITY, l_row = 0.f;
            {
                uint32_t x[32];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    tmem_ld32(tX + c * 32, x);
                    tmem_wait_ld();
                    if (all_vis) {
#pragma unroll
                        for (int t = 0; t < 32; ++t) m_row = fmaxf(m_row, __uint_as_float(x[t]));
                    } else {
                        const uint32_t vw = my_vis ? (c == 0 ? vw0 : c == 1 ? vw1 : c == 2 ? vw2 : vw3) : 0u;
#pragma unroll
                        for (int t = 0; t < 32; ++t)
                            if ((vw >> t) & 1u) m_row = fmaxf(m_row, __uint_as_float(x[t]));
                    }
                }
                const float mc = (my_vis ? m_row : 0.f) * c2;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    tmem_ld32(tX + c * 32, x);
                    tmem_wait_ld();
                    const uint32_t vw = my_vis ? (c == 0 ? vw0 : c == 1 ? vw1 : c == 2 ? vw2 : vw3) : 0u;
                    uint32_t pk[16];
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float e0 = fast_exp2(fmaf(__uint_as_float(x[t]), c2, -mc));
                        float e1 = fast_exp2(fmaf(__uint_as_float(x[t + 1]), c2, -mc));
                        if (!all_vis) {
                            if (!((vw >> t) & 1u)) e0 = 0.f;
                            if (!((vw >> (t + 1)) & 1u)) e1 = 0.f;
                        }
                        l_row += e0 + e1;
                        pk[t >> 1] = pack_bf16x2(e0, e1);
                    }
                    tmem_st16(tX + c * 16, pk);
                }
            }
            tmem_wait_st();
            // warp maximum of the row maxima, for the joint-softmax merge
            float m_w = m_row;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) m_w = fmaxf(m_w, __shfl_xor_sync(0xFFFFFFFFu, m_w, o));
            if (lane == 0) sMpart[warp] = m_w;
            tc_fence_before();
            __syncthreads();                                           // B3
            if (warp == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < RING / 16; ++kk)
                    umma_ts_pred(tmem_base + 128, tmem_base + kk * 8, dVsM + kk * (2048 / 16), idesc_u, kk > 0, issuer);
                umma_commit_pred(bar, issuer);
                if (lane == 0 && !mbar_wait(bar, phase)) *sFail = 1;
                __syncwarp();
            }
            phase ^= 1;
            const float M = fmaxf(fmaxf(sMpart[0], sMpart[1]), fmaxf(sMpart[2], sMpart[3]));
            const float w_row = my_vis ? fast_exp2((m_row - M) * c2) : 0.f;
            __syncthreads();                                           // B4
            tc_fence_after();
            if (*sFail) { failed = true; break; }

            // --- epilogue: Y[d] = sum_j w_j Vr_j[d] U[j][d] / L ---------------------
            {
                uint32_t u[32];
                float v[32];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    tmem_ld32(tU + c * 32, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        const float2 vr = unpack_bf16x2(rVr[c * 16 + (t >> 1)]);
                        v[t] = w_row * vr.x * __uint_as_float(u[t]);
                        v[t + 1] = w_row * vr.y * __uint_as_float(u[t + 1]);
                    }
                    const float s = warp_transpose_sum(v, lane);
                    sRed[warp * (D + 4) + c * 32 + lane] = s;
                }
                float wl = w_row * l_row;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) wl += __shfl_xor_sync(0xFFFFFFFFu, wl, o);
                if (lane == 0) sRed[warp * (D + 4) + D] = wl;
            }
            if (tid < CH) asm volatile("cp.async.wait_all;" ::: "memory");
            tc_fence_before();
            __syncthreads();                                           // B5
            {
                const float Lsum = sRed[D] + sRed[(D + 4) + D] + sRed[2 * (D + 4) + D] + sRed[3 * (D + 4) + D];
                if (tid < D) {
                    const float y = sRed[tid] + sRed[(D + 4) + tid] + sRed[2 * (D + 4) + tid] + sRed[3 * (D + 4) + tid];
                    p.Y[row * D + tid] = __float2bfloat16(y / Lsum);
                }
                if (tid == 0) { p.m[row] = M * p.scale; p.l[row] = Lsum; }
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace sgring
