// Windowed single-gather forward for sm_100a ("ring" schedule, role-specialised and pipelined).
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
//  * Per (query, head):  X = (Q_i o R) S^T  is one 128x128xD product with the
//    Hadamard tile built in shared memory; the E warps take the maximum M over
//    the whole tile (the softmax is joint over (j,k)) and the two threads of row j
//    write P = exp2((x - M) c2) back to tensor memory as BF16 over score columns
//    they have consumed themselves; U = P Vs is the second product with A read
//    from tensor memory and the Vs ring as an MN-major B operand; the epilogue
//    collapses  sum_j Vr_j o U_j  with warp shuffles and divides by L = sum P.
//  * The score scale is folded into the exp2 argument, so the only BF16
//    rounding before the score MMA is the product Q_i[d] * R_j[d] itself.
//
// Schedule.  Tensor memory holds two (X, U) pairs, so two heads are in flight:
//
//   H warps (4)  build Qp = Q_i o R (one ring row per thread, two buffers), prefetch the rows of
//                the key that enters the window next and replace the S ring row.
//   MMA warp (1) issues X(n) = Qp(n) S^T, then U(n-1) = P(n-1) Vs, so the score product of the
//                next head runs while the E warps still work on this one.
//   E warps (8)  thread (row j, column half c): maximum of its half row, joint maximum M over the CTA,
//                P = exp2((x - M) c2) and its sum; then, one head behind, the epilogue of
//                U(n-1).  They also replace the Vs ring row, behind the last U product that reads it.
//
// Hand-offs (mbarriers, one per buffer b = n & 1, phase = (n >> 1) & 1):
//   Qp_full[b]  H -> MMA    tile written (and the S ring row current)
//   X_done[b]   MMA -> E,H  scores in tensor memory; Qp[b] and the S ring read
//   P_full[b]   E -> MMA    P stored (and the Vs ring row current)
//   U_done[b]   MMA -> E    U in tensor memory; P(n) and the Vs ring read
//   U_free[b]   E -> MMA    U(n) taken out of tensor memory
//   Next_ready  H -> E      per query boundary: the prefetched rows of the entering key have landed
// The E warps also meet each other on mbarriers rather than named barriers, so that these waits are
// bounded like the rest, and both meetings are split so that nobody stands waiting: the warps post
// their maxima before the epilogue of the previous head and pick the joint maximum up after it; the
// output reduction of head m is finished at the start of the epilogue of head m + 1.
// Every wait is bounded and watches a CTA-wide failure flag (status code instead of a hang).
#pragma once

#include <cuda.h>

#include "sg_ring_common.cuh"

namespace sgring {

struct FwdParams {
    const __nv_bfloat16* Q;        // [B,Hq,N,D]
    const __nv_bfloat16* R;        // [B,Hkv,N,D]
    const __nv_bfloat16* S;
    const __nv_bfloat16* Vr;
    const __nv_bfloat16* Vs;
    const uint8_t* mask;           // [B,N,N] or null
    const uint32_t* mask_words;    // the same mask as packed words [B,N,ceil(N/32)], or null (takes precedence)
    __nv_bfloat16* Y;              // [B,Hq,N,D]
    float* m;                      // [B,Hq,N]
    float* l;
    int B, Hq, Hkv, N, window, q_begin, block_len;
    int bnhd;                      // memory layout of Q, R, S, Vr, Vs, Y: 0 [B,H,N,D], 1 [B,N,H,D] (RowAddr)
    __nv_bfloat16* Y_act;          // optional second output QuickGELU(Y) = Y * sigmoid(1.702 Y), laid out like Y; or null
    int precise;                   // 1: the score product runs on Q o R split into its BF16 value and the exact BF16 residual
    int window_s;                  // window on the S / Vs key axis (`window` is the R / Vr axis's); equal unless asymmetric
    float scale;
    int* status;                   // device status word (bounded-wait failures)
    // TMA descriptors (box = one row) over Q viewed as [B*Hq*N, D] and R, Vr, S, Vs viewed as [B*Hkv*N, D]
    CUtensorMap tmQ, tmR, tmVr, tmS, tmVs;
};

enum FwdBar {
    FB_QP_FULL0 = 0, FB_QP_FULL1, FB_X_DONE0, FB_X_DONE1, FB_P_FULL0, FB_P_FULL1, FB_U_DONE0, FB_U_DONE1,
    FB_U_FREE0, FB_U_FREE1, FB_H_SYNC, FB_M_SYNC, FB_STAGE0, FB_STAGE1,
    FB_E_SYNC, FB_NEXT_READY0, FB_COUNT = FB_NEXT_READY0 + 8
};

// The H warps can be up to five query boundaries ahead of the E warps' ring update (two tile buffers,
// two score buffers and the product kept back), so the prefetched rows and their ready flags are
// kept eight deep: neither a buffer nor a barrier phase comes round again before it is consumed.
constexpr int NEXT_BUFS = 8;

template <int D>
struct FwdSmem {
    static constexpr int TILE = RING * D * 2;           // bytes of one [128][D] BF16 tile
    static constexpr int OFF_S = 0;
    static constexpr int OFF_VS = TILE;
    static constexpr int OFF_QP = 2 * TILE;             // 2 buffers
    static constexpr int OFF_QSTAGE = 4 * TILE;         // 2 x D bf16
    static constexpr int NEXT_BYTES = 4 * D * 2;        // rows R, Vr, S, Vs of an entering key
    static constexpr int OFF_NEXT = OFF_QSTAGE + 2 * D * 2;          // NEXT_BUFS buffers (query index mod NEXT_BUFS)
    static constexpr int OFF_RED = OFF_NEXT + NEXT_BUFS * NEXT_BYTES;        // 2 x 4 x (D + 4) floats: y partials, l partials
    static constexpr int OFF_MPART = OFF_RED + 2 * 4 * (D + 4) * 4;  // 2 x 8 floats: warp maxima, per head parity
    static constexpr int OFF_BARS = OFF_MPART + 2 * 8 * 4;
    static constexpr int OFF_MISC = OFF_BARS + FB_COUNT * 8;         // tmem slot (4) + fail flag (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;          // slack for manual 1024-byte alignment
};

// EXT = false compiles the plain call (layout [B,H,N,D], one window, byte mask, no activated output) with the
// extension fields folded to constants: the role loops are sensitive to every live register, and the plain
// call is the common one.
template <int D, bool EXT = false>
__global__ void __launch_bounds__(PIPE_THREADS, 1) sg_ring_fwd_kernel(const __grid_constant__ FwdParams p) {
    const int x_bnhd = EXT ? p.bnhd : 0;
    const int x_window_s = EXT ? p.window_s : p.window;
    __nv_bfloat16* const x_Y_act = EXT ? p.Y_act : nullptr;
    const uint32_t* const x_mask_words = EXT ? p.mask_words : nullptr;
    const bool x_precise = EXT && p.precise != 0;
    using L = FwdSmem<D>;
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int DW = D / 2;            // packed bf16x2 words per row
    constexpr int HD = D / 2;            // output columns per E thread
    constexpr uint32_t TMEM_COLS = 512;  // buffer b: X/P at b*256, U at b*256 + 128
    constexpr int E_REGS = 120, H_REGS = 152, M_REGS = 96;
    static_assert(8 * E_REGS + 4 * H_REGS + 4 * M_REGS <= 2048, "register file: 64K registers / 32 lanes");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sS = smem + L::OFF_S;
    uint8_t* sVs = smem + L::OFF_VS;
    uint8_t* sQp = smem + L::OFF_QP;
    __nv_bfloat16* sQst = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_QSTAGE);
    uint8_t* sNext = smem + L::OFF_NEXT;
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    float* sMpart = reinterpret_cast<float*>(smem + L::OFF_MPART);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + blockIdx.x * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const bool is_h = warp >= 8 && warp < 12, is_mma = warp == 12;

    if (is_mma) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        // Arrival counts are in warps: one elected lane arrives for its warp (warp_arrive).
        for (int x = 0; x < 2; ++x) {
            mbar_init(&bars[FB_QP_FULL0 + x], 4);
            mbar_init(&bars[FB_X_DONE0 + x], 1);
            mbar_init(&bars[FB_P_FULL0 + x], 8);
            mbar_init(&bars[FB_U_DONE0 + x], 1);
            mbar_init(&bars[FB_U_FREE0 + x], 8);
        }
        mbar_init(&bars[FB_H_SYNC], 4);
        // staging barriers: one arrival (the issuing thread's expect_tx) plus the bytes the TMA copies deliver
        for (int x = 0; x < NEXT_BUFS; ++x) mbar_init(&bars[FB_NEXT_READY0 + x], 1);
        mbar_init(&bars[FB_STAGE0], 1);
        mbar_init(&bars[FB_STAGE1], 1);
        mbar_init(&bars[FB_M_SYNC], 8);
        mbar_init(&bars[FB_E_SYNC], 8);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;       // statistics-style row index of key 0
    const RowAddr kaddr{x_bnhd, p.Hkv, p.N, D};
    const size_t kstep = kaddr.step();                                       // elements from one key's row to the next
    const __nv_bfloat16* gR = p.R + kaddr.elem(kv_base);
    const __nv_bfloat16* gS = p.S + kaddr.elem(kv_base);
    const __nv_bfloat16* gVr = p.Vr + kaddr.elem(kv_base);
    const __nv_bfloat16* gVs = p.Vs + kaddr.elem(kv_base);
    const MaskView mask_b = mask_view(p.mask, x_mask_words, b, p.N);
    const int n_iter = (q1 - q0) * G;
    auto row_at = [&](int i, int hh) {
        return (static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i;
    };
    auto next_row = [&](int i, int hh) { return hh + 1 < G ? row_at(i, hh + 1) : row_at(i + 1, 0); };
    // Element offset of the row of (position i, head hh of this KV group) in Q, dY, Y, dQ, its tensor-map coordinates,
    // and the coordinates of a key's row (RowAddr describes the two layouts; here without its divisions).
    auto qoff_at = [&](int i, int hh) -> size_t {
        return x_bnhd ? ((static_cast<size_t>(b) * p.N + i) * p.Hq + (g * G + hh)) * D
                      : ((static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i) * D;
    };
    auto q_tma = [&](int i, int hh, int& x, int& y) {
        if (x_bnhd) { x = (g * G + hh) * D; y = b * p.N + i; }
        else { x = 0; y = (b * p.Hq + (g * G + hh)) * p.N + i; }
    };
    auto k_tma = [&](int key, int& x, int& y) {
        if (x_bnhd) { x = g * D; y = b * p.N + key; }
        else { x = 0; y = static_cast<int>(kv_base) + key; }
    };
    const size_t qstep = x_bnhd ? static_cast<size_t>(p.Hq) * D : D;      // elements between consecutive positions of one head
    const float c2 = p.scale * LOG2E;

    uint32_t tmem_base = 0;
    auto cta_start_sync = [&]() {
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        tmem_base = *tmem_slot;
    };

    if (is_h) {
        // ================================================================== H warps
        reg_inc<H_REGS>();
        const int hslot = tid - PIPE_E_THREADS;          // ring slot of this thread
        uint32_t rR[DW];
        {   // initial fill: R row in registers, S and Vs rows in the operand tiles
            const int key = ring_key(q0, hslot);
            if (key >= 0) {
                const uint4* r4 = reinterpret_cast<const uint4*>(gR + static_cast<size_t>(key) * kstep);
                const uint4* s4 = reinterpret_cast<const uint4*>(gS + static_cast<size_t>(key) * kstep);
                const uint4* vs4 = reinterpret_cast<const uint4*>(gVs + static_cast<size_t>(key) * kstep);
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const uint4 a = __ldg(r4 + c);
                    rR[4 * c] = a.x; rR[4 * c + 1] = a.y; rR[4 * c + 2] = a.z; rR[4 * c + 3] = a.w;
                    *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(hslot, c)) = __ldg(s4 + c);
                    *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(hslot, c)) = __ldg(vs4 + c);
                }
            } else {
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    rR[4 * c] = rR[4 * c + 1] = rR[4 * c + 2] = rR[4 * c + 3] = 0;
                    *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(hslot, c)) = z;
                    *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(hslot, c)) = z;
                }
            }
        }
        // Row staging by TMA, issued by one thread: the Q row of iteration `it` into its stage buffer and, when
        // next_key >= 0, the four rows (R, Vr, S, Vs) of the key that enters the ring with query next_key.
        // Each copy names an mbarrier that counts its bytes; the consumers wait on that barrier.
        auto h_stage = [&](int it, int qi, int qh, int next_key) {
            if (hslot != 0) return;
            if (it >= 0) {
                uint64_t* bar = &bars[FB_STAGE0 + (it & 1)];
                mbar_arrive_expect_tx(bar, D * 2);
                int x, y;
                q_tma(qi, qh, x, y);
                tma_load_2d(sQst + (it & 1) * D, &p.tmQ, x, y, bar);
            }
            if (next_key >= 0) {
                uint64_t* bar = &bars[FB_NEXT_READY0 + ((next_key - q0 - 1) & (NEXT_BUFS - 1))];
                uint8_t* dst = sNext + (next_key & (NEXT_BUFS - 1)) * L::NEXT_BYTES;
                int kx, krow;
                k_tma(next_key, kx, krow);
                mbar_arrive_expect_tx(bar, 4 * D * 2);
                tma_load_2d(dst, &p.tmR, kx, krow, bar);
                tma_load_2d(dst + D * 2, &p.tmVr, kx, krow, bar);
                tma_load_2d(dst + 2 * D * 2, &p.tmS, kx, krow, bar);
                tma_load_2d(dst + 3 * D * 2, &p.tmVs, kx, krow, bar);
            }
        };
        fence_async_smem();
        cta_start_sync();
        h_stage(0, q0, 0, -1);
        constexpr int HB = 8;                 // staged chunks in flight per thread
        int n = 0, it = 0;
        bool ok = true;
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            const int s = i & (RING - 1);
            uint32_t vw[4];
            ring_visibility(mask_b.row(i), i, min(p.window, x_window_s), lane, vw);      // a pair needs a key on both axes
            const bool work = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                // The staged Q row of this iteration has landed (TMA byte counts; the issuing warp looks, the
                // others learn it through H_sync, which that warp joins afterwards); everyone is past the
                // previous build.
                const bool boundary = hh == 0 && i > q0;      // key i replaces key i-128 in slot s
                if (warp == 8) {
                    ok = pipe_wait<true>(&bars[FB_STAGE0 + (it & 1)], (it >> 1) & 1, sFail, 13);
                    if (ok && boundary) {
                        const int fb = i - q0 - 1;            // the entering key's rows were requested one query ago
                        ok = pipe_wait<true>(&bars[FB_NEXT_READY0 + (fb & (NEXT_BUFS - 1))], (fb >> 3) & 1, sFail, 14);
                    }
                }
                warp_arrive(&bars[FB_H_SYNC], lane);
                ok = ok & pipe_wait<true>(&bars[FB_H_SYNC], it & 1, sFail, 10);
                if (!ok) break;
                const uint8_t* nx = sNext + (i & (NEXT_BUFS - 1)) * L::NEXT_BYTES;
                if (boundary && hslot == s) {
                    const uint4* r4 = reinterpret_cast<const uint4*>(nx);
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        const uint4 a = r4[c];
                        rR[4 * c] = a.x; rR[4 * c + 1] = a.y; rR[4 * c + 2] = a.z; rR[4 * c + 3] = a.w;
                    }
                }
                if (it + 1 < n_iter)
                    h_stage(it + 1, hh + 1 < G ? i : i + 1, hh + 1 < G ? hh + 1 : 0, (hh == 0 && i + 1 < q1) ? i + 1 : -1);
                const int qb = n & 1;
                if (work) {
                    // Qp[n&1] was last read by the score MMAs of head n-2.  In the compensated mode a head fills both
                    // buffers (value, residual), which the score MMAs of head n-1 were the last to read.
                    if (!x_precise) { if (n >= 2) ok = pipe_wait<true>(&bars[FB_X_DONE0 + qb], ((n >> 1) - 1) & 1, sFail, 11); }
                    else if (n >= 1) ok = pipe_wait<true>(&bars[FB_X_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, 11);
                    if (!ok) break;
                    uint8_t* dQp = sQp + (x_precise ? 0 : qb) * L::TILE;
                    const uint4* q4 = reinterpret_cast<const uint4*>(sQst + (it & 1) * D);
                    // The staged row is read in batches ahead of the stores: the compiler cannot tell that the
                    // tile stores do not alias the staging area and would otherwise serialise per chunk.
#pragma unroll
                    for (int c0 = 0; c0 < CH; c0 += HB) {
                        uint4 q[HB];
#pragma unroll
                        for (int c = 0; c < HB; ++c) q[c] = q4[c0 + c];
#pragma unroll
                        for (int c = 0; c < HB; ++c) {
                            uint4 o;
                            o.x = mul_bf16x2(q[c].x, rR[4 * (c0 + c)]);
                            o.y = mul_bf16x2(q[c].y, rR[4 * (c0 + c) + 1]);
                            o.z = mul_bf16x2(q[c].z, rR[4 * (c0 + c) + 2]);
                            o.w = mul_bf16x2(q[c].w, rR[4 * (c0 + c) + 3]);
                            st_shared_v4(dQp + sw128_offset<RING>(hslot, c0 + c), o.x, o.y, o.z, o.w);
                            if (EXT && x_precise) {
                                uint4 lo;
                                lo.x = mul_residual_bf16x2(q[c].x, rR[4 * (c0 + c)], o.x);
                                lo.y = mul_residual_bf16x2(q[c].y, rR[4 * (c0 + c) + 1], o.y);
                                lo.z = mul_residual_bf16x2(q[c].z, rR[4 * (c0 + c) + 2], o.z);
                                lo.w = mul_residual_bf16x2(q[c].w, rR[4 * (c0 + c) + 3], o.w);
                                *reinterpret_cast<uint4*>(dQp + L::TILE + sw128_offset<RING>(hslot, c0 + c)) = lo;
                            }
                        }
                    }
                }
                if (boundary) {
                    // The S row of slot s changes key once every score MMA issued so far is complete (the
                    // last one is head n-1; this thread waits for the same phase again when it reuses
                    // that tile buffer).
                    if (n >= 1) ok = pipe_wait<true>(&bars[FB_X_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, 12);
                    if (!ok) break;
                    if (hslot < CH)
                        *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(s, hslot)) =
                            *reinterpret_cast<const uint4*>(nx + 2 * (D * 2) + hslot * 16);
                }
                if (work || boundary) fence_async_smem();
                if (work) {
                    warp_arrive(&bars[FB_QP_FULL0 + qb], lane);
                    ++n;
                }
            }
        }
    } else if (warp >= 12) {
        reg_dec<M_REGS>();
        cta_start_sync();
        if (is_mma) {
        // ================================================================== MMA warp
        // The whole warp runs this role converged; MMAs and commits are predicated on one elected lane.
        const uint32_t issuer = elect_one();
        const uint32_t idesc_x = make_idesc_bf16(RING, RING, 0, 0);
        const uint32_t idesc_u = make_idesc_bf16(RING, D, 0, 1);
        const uint64_t dQp = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);           // A, K-major
        const uint64_t dS = make_smem_desc(smem_u32(sS), 16, 1024, SWIZZLE_128B);             // B, K-major
        const uint64_t dVsM = make_smem_desc(smem_u32(sVs), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major
        int n = 0;
        bool ok = true, u_pending = false;
        // U(m) = P(m) Vs.  P sits in the score columns: thread (row, half c) keeps its 32 packed columns
        // at the start of its own 64, so k-step kk reads columns 64*(kk/4) + 8*(kk%4).
        auto issue_u = [&](int m) {
            const int ub = m & 1;
            bool r = pipe_wait<true>(&bars[FB_P_FULL0 + ub], (m >> 1) & 1, sFail, 22);
            if (r && m >= 2) r = pipe_wait<true>(&bars[FB_U_FREE0 + ub], ((m >> 1) - 1) & 1, sFail, 23);
            if (r) {
                tc_fence_after();
                const uint32_t tX = tmem_base + ub * 256, tU = tX + 128;
#pragma unroll
                for (int kk = 0; kk < RING / 16; ++kk)
                    umma_ts_pred(tU, tX + 64u * (kk >> 2) + 8u * (kk & 3), dVsM + kk * (2048 / 16), idesc_u, kk > 0,
                                 issuer);
                umma_commit_pred(&bars[FB_U_DONE0 + ub], issuer);
            }
            return r;
        };
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            uint32_t vw[4];
            ring_visibility(mask_b.row(i), i, min(p.window, x_window_s), lane, vw);      // a pair needs a key on both axes
            const bool work = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                if (!work) {
                    // nothing follows that would carry the kept-back product: issue it now
                    if (u_pending) { ok = issue_u(n - 1); u_pending = false; }
                    continue;
                }
                const int qb = n & 1;
                ok = pipe_wait<true>(&bars[FB_QP_FULL0 + qb], (n >> 1) & 1, sFail, 20);
                // X[qb] held P(n-2) until the U product of that head had read it
                if (ok && n >= 2) ok = pipe_wait<true>(&bars[FB_U_DONE0 + qb], ((n >> 1) - 1) & 1, sFail, 21);
                if (!ok) break;
                tc_fence_after();
                {
                    const uint32_t tX = tmem_base + qb * 256;
                    const uint64_t dA = dQp + (x_precise ? 0 : qb) * (L::TILE / 16);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                        umma_ss_pred(tX, dA + off, dS + off, idesc_x, kk > 0, issuer);
                    }
                    if (EXT && x_precise) {          // + residual tile: X = (value + residual) S^T
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                            umma_ss_pred(tX, dA + L::TILE / 16 + off, dS + off, idesc_x, 1, issuer);
                        }
                    }
                    umma_commit_pred(&bars[FB_X_DONE0 + qb], issuer);
                }
                if (u_pending) {
                    ok = issue_u(n - 1);
                    if (!ok) break;
                }
                u_pending = true;
                ++n;
            }
        }
        if (ok && u_pending) ok = issue_u(n - 1);
        // the E warps wait for every U product, so nothing is in flight when they are done
        __syncwarp();
        }
    } else {
        // ================================================================== E warps
        reg_dec<E_REGS>();
        cta_start_sync();
        const int slot = tid & (RING - 1);               // tensor-memory lane = ring slot = score row j
        const int ch = tid >> 7;                          // column half of the scores / of the output
        const int quarter = warp & 3;
        const uint32_t tl = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr int VW = HD / 2;                        // packed words of this thread's half of a Vr row
        uint32_t rVr[VW];
        {
            const int key = ring_key(q0, slot);
            if (key >= 0) {
                const uint4* v4 = reinterpret_cast<const uint4*>(gVr + static_cast<size_t>(key) * kstep + ch * HD);
#pragma unroll
                for (int c = 0; c < VW / 4; ++c) {
                    const uint4 v = __ldg(v4 + c);
                    rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int c = 0; c < VW; ++c) rVr[c] = 0;
            }
        }
        // Epilogue of head m, run one head late so that it overlaps the U product:
        //   Y[d] = sum_j Vr_j[d] U[j][d] / L,  L = sum of all P  (P is taken against the joint maximum M,
        //   so the rows need no further weights).
        // Second half of an epilogue, run when the next one starts (or at the end): sum the four lane
        // quarters' partials and write Y, m, l of head fin_m.
        bool fin_pending = false;
        int fin_m = 0;
        size_t fin_row = 0, fin_off = 0;
        float fin_M = 0.f;
        auto finish = [&]() {
            if (!fin_pending) return true;
            fin_pending = false;
            if (!pipe_wait<true>(&bars[FB_E_SYNC], fin_m & 1, sFail, 33)) return false;
            const float* red = sRed + (fin_m & 1) * 4 * (D + 4);
            float Lsum = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) Lsum += red[q * (D + 4) + D] + red[q * (D + 4) + D + 1];
            if (tid < D) {
                const float y = (red[tid] + red[(D + 4) + tid] + red[2 * (D + 4) + tid] + red[3 * (D + 4) + tid]) / Lsum;
                const size_t at = fin_off + tid;
                p.Y[at] = __float2bfloat16(y);
                if (x_Y_act) x_Y_act[at] = __float2bfloat16(y / (1.f + __expf(-1.702f * y)));
            }
            if (tid == 0) { p.m[fin_row] = fin_M * p.scale; p.l[fin_row] = Lsum; }
            return true;
        };
        auto epilogue = [&](int m, size_t row, size_t off, float M, float l_half) {
            const int ub = m & 1;
            if (!finish()) return false;
            bool r = pipe_wait<true>(&bars[FB_U_DONE0 + ub], (m >> 1) & 1, sFail, 32);
            if (!r) return false;
            tc_fence_after();
            const uint32_t tU = tl + ub * 256 + 128 + ch * HD;
            float* red = sRed + ub * 4 * (D + 4);
            constexpr int NC = HD / 32;
#pragma unroll
            for (int c = 0; c < NC; ++c) {      // unrolled: rVr must be indexed with constants to stay in registers
                float s;
                if (EXT && x_precise) {
                    // compensated mode: FP32 products and an FP32 lane sum (no BF16 rounding between U and Y)
                    float va[16], vb[16];
                    {
                        uint32_t u[16];
                        tmem_ld16(tU + c * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int t = 0; t < 16; t += 2) {
                            const float2 vr = unpack_bf16x2(rVr[c * 16 + (t >> 1)]);
                            va[t] = vr.x * __uint_as_float(u[t]);
                            va[t + 1] = vr.y * __uint_as_float(u[t + 1]);
                        }
                    }
                    {
                        uint32_t u[16];
                        tmem_ld16(tU + c * 32 + 16, u);
                        tmem_wait_ld();
                        if (c == NC - 1) {
                            tc_fence_before();
                            warp_arrive(&bars[FB_U_FREE0 + ub], lane);
                        }
#pragma unroll
                        for (int t = 0; t < 16; t += 2) {
                            const float2 vr = unpack_bf16x2(rVr[c * 16 + 8 + (t >> 1)]);
                            vb[t] = vr.x * __uint_as_float(u[t]);
                            vb[t + 1] = vr.y * __uint_as_float(u[t + 1]);
                        }
                    }
                    s = warp_transpose_sum_2x16(va, vb, lane);
                } else {
                    // two rounds of 16 columns keep the live set small.  U is rounded to BF16 pairs and multiplied by the
                    // packed Vr words as they are: two instructions a pair, and the lane sum below wants BF16 pairs anyway
                    uint32_t w[16];
                    {
                        uint32_t u[16];
                        tmem_ld16(tU + c * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int t = 0; t < 16; t += 2)
                            w[t >> 1] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[t]), __uint_as_float(u[t + 1])),
                                                   rVr[c * 16 + (t >> 1)]);
                    }
                    {
                        uint32_t u[16];
                        tmem_ld16(tU + c * 32 + 16, u);
                        tmem_wait_ld();
                        if (c == NC - 1) {
                            // U is in registers: the product of head m + 2 may overwrite it
                            tc_fence_before();
                            warp_arrive(&bars[FB_U_FREE0 + ub], lane);
                        }
#pragma unroll
                        for (int t = 0; t < 16; t += 2)
                            w[8 + (t >> 1)] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[t]), __uint_as_float(u[t + 1])),
                                                         rVr[c * 16 + 8 + (t >> 1)]);
                    }
                    // (a shared-memory transpose for this lane sum was measured slower: it competes with the
                    //  MMA operand reads for shared-memory bandwidth)
                    s = warp_transpose_sum_words(w, lane);
                }
                red[quarter * (D + 4) + ch * HD + c * 32 + lane] = s;
            }
            float wl = l_half;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) wl += __shfl_xor_sync(0xFFFFFFFFu, wl, o);
            if (lane == 0) red[quarter * (D + 4) + D + ch] = wl;
            warp_arrive(&bars[FB_E_SYNC], lane);
            fin_pending = true; fin_m = m; fin_row = row; fin_off = off; fin_M = M;
            return true;
        };
        // Key i takes over slot s: the Vs ring row (every U product that read the old row is complete,
        // because the caller has drained its epilogues) and this thread's half of the Vr row.
        auto ring_update = [&](int i) {
            const int s = i & (RING - 1), fb = i - q0 - 1;
            const uint8_t* nx = sNext + (i & (NEXT_BUFS - 1)) * L::NEXT_BYTES;
            if (!pipe_wait<true>(&bars[FB_NEXT_READY0 + (fb & (NEXT_BUFS - 1))], (fb >> 3) & 1, sFail, 34)) return false;
            if (tid < CH)
                *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(s, tid)) =
                    *reinterpret_cast<const uint4*>(nx + 3 * (D * 2) + tid * 16);
            if (slot == s) {
                const uint4* v4 = reinterpret_cast<const uint4*>(nx + D * 2 + ch * HD * 2);
#pragma unroll
                for (int c = 0; c < VW / 4; ++c) {
                    const uint4 v = v4[c];
                    rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                }
            }
            fence_async_smem();
            return true;
        };
        int n = 0;
        bool ok = true, pend = false;
        int pend_n = 0;
        size_t pend_row = 0, pend_off = 0;
        float pend_m = 0.f, pend_l = 0.f;
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            // rows of the score tile are R keys (window), columns S keys (window_s)
            uint32_t vw[4], vs[4];
            ring_visibility(mask_b.row(i), i, p.window, lane, vw);
            if (x_window_s != p.window) ring_visibility(mask_b.row(i), i, x_window_s, lane, vs);
            else { vs[0] = vw[0]; vs[1] = vw[1]; vs[2] = vw[2]; vs[3] = vw[3]; }
            const int n_rows = __popc(vw[0]) + __popc(vw[1]) + __popc(vw[2]) + __popc(vw[3]);
            const int n_cols = __popc(vs[0]) + __popc(vs[1]) + __popc(vs[2]) + __popc(vs[3]);
            const bool live = min(n_rows, n_cols) != 0;          // false: no visible pair
            const bool all_vis = n_rows == RING && n_cols == RING;
            const bool my_vis = (vw[quarter] >> lane) & 1u;
            // visibility words of this thread's two 32-column chunks
            const uint32_t cw0 = my_vis ? (ch ? vs[2] : vs[0]) : 0u;
            const uint32_t cw1 = my_vis ? (ch ? vs[3] : vs[1]) : 0u;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                const size_t row = row_at(i, hh);
                const bool boundary = hh == 0 && i > q0;
                const int xb = n & 1;
                const uint32_t tX = tl + xb * 256 + ch * 64;          // this thread's 64 score columns
                if (live) {
                    ok = pipe_wait<true>(&bars[FB_X_DONE0 + xb], (n >> 1) & 1, sFail, 30);
                    if (!ok) break;
                    tc_fence_after();
                    // ---- maximum of this thread's half row; the other half belongs to the thread with the same
                    //      lane in the partner warp, and the exchange completes behind the epilogue below
                    // four independent running maxima: one chain of 64 dependent max operations would cost
                    // more than the loads
                    float mh0 = -INFINITY, mh1 = -INFINITY, mh2 = -INFINITY, mh3 = -INFINITY;
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t x[32];
                        tmem_ld32(tX + cc * 32, x);
                        tmem_wait_ld();
                        const uint32_t cw = cc ? cw1 : cw0;
                        if (all_vis) {
#pragma unroll
                            for (int t = 0; t < 32; t += 8) {
                                mh0 = fmaxf(mh0, fmaxf(__uint_as_float(x[t]), __uint_as_float(x[t + 1])));
                                mh1 = fmaxf(mh1, fmaxf(__uint_as_float(x[t + 2]), __uint_as_float(x[t + 3])));
                                mh2 = fmaxf(mh2, fmaxf(__uint_as_float(x[t + 4]), __uint_as_float(x[t + 5])));
                                mh3 = fmaxf(mh3, fmaxf(__uint_as_float(x[t + 6]), __uint_as_float(x[t + 7])));
                            }
                        } else {
#pragma unroll
                            for (int t = 0; t < 32; t += 4) {
                                if ((cw >> t) & 1u) mh0 = fmaxf(mh0, __uint_as_float(x[t]));
                                if ((cw >> (t + 1)) & 1u) mh1 = fmaxf(mh1, __uint_as_float(x[t + 1]));
                                if ((cw >> (t + 2)) & 1u) mh2 = fmaxf(mh2, __uint_as_float(x[t + 2]));
                                if ((cw >> (t + 3)) & 1u) mh3 = fmaxf(mh3, __uint_as_float(x[t + 3]));
                            }
                        }
                    }
                    const float mh = fmaxf(fmaxf(mh0, mh1), fmaxf(mh2, mh3));
                    {
                        float m_w = mh;
#pragma unroll
                        for (int o = 16; o >= 1; o >>= 1) m_w = fmaxf(m_w, __shfl_xor_sync(0xFFFFFFFFu, m_w, o));
                        if (lane == 0) sMpart[xb * 8 + warp] = m_w;
                    }
                    warp_arrive(&bars[FB_M_SYNC], lane);
                }
                // ---- epilogue of the previous head, behind its U product; then the ring rows of a new key
                if (pend) { ok = epilogue(pend_n, pend_row, pend_off, pend_m, pend_l); pend = false; }
                if (ok && boundary) ok = ring_update(i);
                if (!ok) break;
                if (!live) {
                    // No visible pair: Y = 0, m = NEG_INF, l = 0 (cuda/common.cuh:24).
                    if (tid < D) {
                        p.Y[qoff_at(i, hh) + tid] = __float2bfloat16(0.f);
                        if (x_Y_act) x_Y_act[qoff_at(i, hh) + tid] = __float2bfloat16(0.f);
                    }
                    if (tid == 0) { p.m[row] = NEG_INF_F; p.l[row] = 0.f; }
                    continue;
                }
                ok = pipe_wait<true>(&bars[FB_M_SYNC], n & 1, sFail, 31);
                if (!ok) break;
                const float* mp = sMpart + xb * 8;
                const float M = fmaxf(fmaxf(fmaxf(mp[0], mp[1]), fmaxf(mp[2], mp[3])),
                                      fmaxf(fmaxf(mp[4], mp[5]), fmaxf(mp[6], mp[7])));
                const float mc = M * c2;
                // ---- P = exp2((x - M) c2), BF16 over the first 32 of this thread's columns; half-row sum
                // packed FP32 arithmetic: one instruction for the exponents of two columns, one for their sums
                const uint64_t c2p = pair_f32(c2, c2), mcp = pair_f32(-mc, -mc);
                uint64_t ls0 = pair_f32(0.f, 0.f), ls1 = ls0;          // two independent chains of partial sums
#pragma unroll 1
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t x[32], pk[16];
                    tmem_ld32(tX + cc * 32, x);
                    tmem_wait_ld();
                    const uint32_t cw = cc ? cw1 : cw0;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float a0, a1;
                        unpair_f32(fma_f32x2(pair_b32(x[t], x[t + 1]), c2p, mcp), a0, a1);
                        float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
                        if (!all_vis) {
                            if (!((cw >> t) & 1u)) e0 = 0.f;
                            if (!((cw >> (t + 1)) & 1u)) e1 = 0.f;
                        }
                        if (t & 2) ls1 = add_f32x2(ls1, pair_f32(e0, e1));
                        else ls0 = add_f32x2(ls0, pair_f32(e0, e1));
                        pk[t >> 1] = pack_bf16x2(e0, e1);
                    }
                    tmem_st16(tX + cc * 16, pk);
                }
                float l_half;
                {
                    float s0, s1;
                    unpair_f32(add_f32x2(ls0, ls1), s0, s1);
                    l_half = s0 + s1;
                }
                tmem_wait_st();
                tc_fence_before();
                // P_full also tells the MMA warp that the Vs ring row is current (ring_update above)
                warp_arrive(&bars[FB_P_FULL0 + xb], lane);
                pend = true; pend_n = n; pend_row = row; pend_off = qoff_at(i, hh); pend_m = M; pend_l = l_half;
                ++n;
            }
        }
        if (ok && pend) ok = epilogue(pend_n, pend_row, pend_off, pend_m, pend_l);
        if (ok) ok = finish();
    }
    tc_fence_before();
    __syncthreads();
    if (*sFail && tid == 0) atomicExch(p.status, 100 + *sFail);
    if (is_mma) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace sgring
