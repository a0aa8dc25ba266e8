// Windowed single-gather backward for sm_100a ("ring" schedule, role-specialised and pipelined).
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
//      and stores both to tensor memory as BF16 over the score columns it has consumed itself
//      dKb += gA^T (Q_i o Ka),  dVb += P^T (dY_i o Va)          A from tensor memory,
//                                                              B = the Hadamard tiles (MN-major)
//      dQ pass only:  W = gA^T Ka, then dQ_i = scale * sum_k Kb_k o W_k by warp shuffles.
//    The forward statistics (m, l) make P purely elementwise, so no row reduction
//    is needed here.
//  * When query i reuses slot i mod 128 the lane holding key i-128 is final for
//    this CTA: it is copied to an FP32 partial buffer and zeroed (by the flush warp of that lane quarter).  Query
//    block x writes partial plane x mod P with P large enough that blocks sharing a
//    plane touch disjoint key rows (bwd_planes), so every partial row has exactly
//    one writer and the final sum (reduce kernel below) has a fixed order: repeated
//    calls are bit-identical.
//
// Schedule.  Tensor memory holds the two accumulators (2 x 128 columns) and two 128-column
// regions R0, R1 for everything transient, so only one head's P^T/gA^T can be live at a time;
// what overlaps is the next head's score product and exponentials with this head's
// accumulation.  Head n uses A(n) = R[n & 1] for X^T -> P^T, gA^T and B(n) = R[~n & 1] for
// dP^T (then W in the dQ pass), so the regions swap roles every head:
//
//   H warps (4)  build the Hadamard tiles Qp = Q_i o Ka, Gt = dY_i o Va (one ring row per
//                thread, double-buffered), replace the ring row of the key that leaves the
//                window (its rows are prefetched a query ahead), and flush + zero the
//                accumulator lane of that key.
//   MMA warp (1) one thread issues, for head n:
//                  X^T(n) -> A(n)      as soon as B(n-1) has been read by the E warps
//                  dKb += gA^T(n-1) Qp (kept back until here when there is no dQ to form)
//                  dP^T(n) -> B(n)     once head n-1's accumulation has read A(n-1) = B(n)
//                  dVb += P^T(n) Gt
//                  dQ pass: W(n) = gA^T(n) Ka -> B(n), then dKb += gA^T(n) Qp
//   E warps (8)  thread (lane k, column half c): P^T = exp2(X^T c2 - lse) for its 64 columns,
//                stored as BF16 over the first 32 of them; gA^T = P^T o (dP^T - delta) over
//                the other 32 (so no E thread writes columns another one still reads);
//                dQ pass: collapse W to dQ.
//
// Hand-offs (mbarriers; phase = processed-head counter unless noted):
//   Qp_full[b], Gt_full[b]  H -> MMA  tile buffer b written   D_done[b]  MMA -> H,MMA  dKb MMAs of buffer b done
//   S_xt,S_dp  MMA -> E   X^T / dP^T in tensor memory    P_full,G_full  E -> MMA  P^T / gA^T stored
//   B_free     E -> MMA   B(n) read (dP^T, or W)         V_done[b]  MMA -> H   dVb MMAs of Gt buffer b done
//   W_full     MMA -> E   W in tensor memory             Ring_free  MMA(+E) -> H  per query: ring rows read
//   Flush_done H -> MMA   per query: lane flushed        Flush_seen MMA -> H   per query: that was observed
// A waiter observes every phase of a barrier it waits on (a one-bit parity cannot tell phases
// two apart).  Every wait is bounded and also watches a CTA-wide failure flag, so a protocol
// error ends the kernel with a status code instead of hanging it.
#pragma once

#include "sg_ring_common.cuh"

namespace sgring {

// Partial planes.  A block of L queries flushes the key rows (q0 - 128, q1); block x writes plane x mod P.
// Blocks x and x + P then touch disjoint rows iff P * L - 127 >= L, i.e. P >= 127 / L + 1 (rounded up):
// every partial row of a plane has exactly one writer, whatever the block length.
constexpr int BWD_MIN_BLOCK = 16;
__host__ __device__ constexpr int bwd_planes(int block_len) { return (RING - 1 + block_len - 1) / block_len + 1; }

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
    const uint32_t* mask_words;    // the same mask as packed words [B,N,ceil(N/32)], or null (takes precedence)
    const float* delta;              // [B,Hq,N]: rowsum(dY o Y), from the pre-pass (sg_delta_kernel)
    __nv_bfloat16* dQ;               // [B,Hq,N,D], written only by the WITH_DQ instantiation
    float* part_K;                   // [planes][B,Hkv,N,D] FP32 partials of dKb (plane-major)
    float* part_V;                   // [planes][B,Hkv,N,D] FP32 partials of dVb
    int B, Hq, Hkv, N, window, q_begin, block_len, planes;
    int bnhd;                        // memory layout of Q, dY, Y, dQ and the key tensors: 0 [B,H,N,D], 1 [B,N,H,D] (RowAddr)
    int precise;                     // 1: score product on Q o Ka split into its BF16 value and the exact BF16 residual
    int window_oth;                  // window on the other side's key axis (`window` is the own side's); equal unless asymmetric
    float scale;
    int* status;
};

enum PipeBar {
    PB_QP_FULL0 = 0, PB_QP_FULL1, PB_GT_FULL0, PB_GT_FULL1, PB_S_XT, PB_S_DP, PB_P_FULL, PB_G_FULL, PB_D_DONE0, PB_D_DONE1, PB_V_DONE0, PB_V_DONE1,
    PB_W_FULL, PB_B_FREE, PB_E_SYNC2, PB_H_SYNC, PB_RING_FREE, PB_FLUSH_DONE, PB_ACC_DONE, PB_COUNT
};

template <int D, bool WITH_DQ>
struct PipeSmem {
    static constexpr int TILE = RING * D * 2;
    static constexpr int OFF_KB = 0;
    static constexpr int OFF_VB = TILE;
    // Hadamard tiles: Qp is double-buffered so the H warps build the next head while this one
    // is consumed; Gt is double-buffered where shared memory allows (the dQ pass also holds Ka).
    static constexpr int G_BUFS = WITH_DQ ? 1 : 2;
    static constexpr int OFF_QP = 2 * TILE;                        // 2 buffers
    static constexpr int OFF_G = 4 * TILE;                         // G_BUFS buffers
    static constexpr int OFF_KA = 5 * TILE;                        // only WITH_DQ
    static constexpr int OFF_STAGE = 6 * TILE;                     // 2 stages x {Q, dY} rows
    static constexpr int NEXT_BYTES = 4 * D * 2;                   // rows Ka, Va, Kb, Vb of the key that enters next
    static constexpr int OFF_NEXT = OFF_STAGE + 2 * 2 * D * 2;     // 2 buffers (query parity)
    static constexpr int OFF_RED = OFF_NEXT + 2 * NEXT_BYTES;      // 2 x 4 x D floats (dQ partials)
    static constexpr int OFF_BARS = OFF_RED + 2 * 4 * D * 4;
    static constexpr int OFF_MISC = OFF_BARS + PB_COUNT * 8;       // tmem slot (4) + fail flag (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

// Copies a warp's accumulator lanes (only_lane < 0: all 32) to the FP32 partial planes and, on
// request, zeroes them.  Lane k of the accumulators belongs to the key in ring slot k; `tl` is the
// tensor-memory address of the warp's lane quarter, `key` the key of this thread's lane (< 0: none).
template <int D>
__device__ __noinline__ void flush_acc_lanes(uint32_t tl, int lane, int only_lane, int key, float* part_k,
                                             float* part_v, float scale, bool rezero) {
    constexpr uint32_t C_AK = 256, C_AV = 384;
    const bool sel = only_lane < 0 || lane == only_lane;
    const bool mine = sel && key >= 0;
    uint32_t a[32];
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const uint32_t col = which ? C_AV : C_AK;
        float* dst_base = which ? part_v : part_k;
        const float mul = which ? 1.0f : scale;
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
                if (sel) {
#pragma unroll
                    for (int t = 0; t < 32; ++t) a[t] = 0;
                }
                tmem_st32(tl + col + c * 32, a);
            }
        }
    }
    if (rezero) {
        tmem_wait_st();
        tc_fence_before();
    }
}

// EXT = false compiles the plain call (layout [B,H,N,D], one window, byte mask) with the extension fields folded
// to constants: the role loops are sensitive to every live register, and the plain call is the common one.
template <int D, bool WITH_DQ, bool EXT = false>
__global__ void __launch_bounds__(PIPE_THREADS, 1) sg_ring_bwd_kernel(const BwdParams p) {
    const int x_bnhd = EXT ? p.bnhd : 0;
    const int x_window_oth = EXT ? p.window_oth : p.window;
    const uint32_t* const x_mask_words = EXT ? p.mask_words : nullptr;
    const bool x_precise = EXT && p.precise != 0;
    using L = PipeSmem<D, WITH_DQ>;
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int DW = D / 2;            // packed words per row
    constexpr int HD = D / 2;            // d columns per E thread in the dQ collapse
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t C_R0 = 0, C_AK = 256, C_AV = 384;   // R1 = R0 + 128

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKb = smem + L::OFF_KB;
    uint8_t* sVb = smem + L::OFF_VB;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sG = smem + L::OFF_G;
    uint8_t* sKa = smem + L::OFF_KA;
    __nv_bfloat16* sStage = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_STAGE);
    uint8_t* sNext = smem + L::OFF_NEXT;
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y;
    const int bx = blockIdx.x;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + bx * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const int parity_buf = bx % p.planes;
    const bool is_h = warp >= 8 && warp < 12, is_mma = warp == 12;

    if (is_mma) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        // Arrival counts are in warps: one elected lane arrives for its warp (warp_arrive).
        mbar_init(&bars[PB_QP_FULL0], 4);   mbar_init(&bars[PB_QP_FULL1], 4);
        mbar_init(&bars[PB_GT_FULL0], 4);   mbar_init(&bars[PB_GT_FULL1], 4);
        mbar_init(&bars[PB_S_XT], 1);       mbar_init(&bars[PB_S_DP], 1);
        mbar_init(&bars[PB_P_FULL], 8);     mbar_init(&bars[PB_G_FULL], 8);
        mbar_init(&bars[PB_D_DONE0], 1);    mbar_init(&bars[PB_D_DONE1], 1);
        mbar_init(&bars[PB_V_DONE0], 1);    mbar_init(&bars[PB_V_DONE1], 1);
        mbar_init(&bars[PB_W_FULL], 1);     mbar_init(&bars[PB_B_FREE], 8);
        mbar_init(&bars[PB_E_SYNC2], 8);    mbar_init(&bars[PB_H_SYNC], 4);
        mbar_init(&bars[PB_RING_FREE], WITH_DQ ? 9 : 1);
        mbar_init(&bars[PB_FLUSH_DONE], 1); mbar_init(&bars[PB_ACC_DONE], 1);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;       // statistics-style row index of key 0
    const RowAddr kaddr{x_bnhd, p.Hkv, p.N, D};
    const size_t kstep = kaddr.step();                                       // elements from one key's row to the next
    const __nv_bfloat16* gKa = p.Ka + kaddr.elem(kv_base);
    const __nv_bfloat16* gVa = p.Va + kaddr.elem(kv_base);
    const __nv_bfloat16* gKb = p.Kb + kaddr.elem(kv_base);
    const __nv_bfloat16* gVb = p.Vb + kaddr.elem(kv_base);
    float* gPartK = p.part_K + (static_cast<size_t>(parity_buf) * p.B * p.Hkv * p.N + kv_base) * D;
    float* gPartV = p.part_V + (static_cast<size_t>(parity_buf) * p.B * p.Hkv * p.N + kv_base) * D;
    const MaskView mask_b = mask_view(p.mask, x_mask_words, b, p.N);

    const int n_iter = (q1 - q0) * G;
    // Row of (query i, head hh of this KV group) in the [B,Hq,N] arrays; the successor of (i, hh) in
    // iteration order is (i, hh + 1) or (i + 1, 0) -- no division by the group size in the loops.
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
    auto next_qoff = [&](int i, int hh) { return hh + 1 < G ? qoff_at(i, hh + 1) : qoff_at(i + 1, 0); };
    const float c2 = p.scale * LOG2E;

    // Each role first sets its register budget (the CTA starts at 128 per thread: the E warps work in
    // rolled rounds of 32 columns and give registers away, the H threads take room for two ring rows
    // and the MMA warp for its descriptors and bookkeeping; 8*E + 4*H + 4*M = 512 registers per lane
    // column), does its share of the set-up and then meets the others at one CTA barrier before the
    // hand-off protocol starts.
    constexpr int E_REGS = 88, H_REGS = 232, M_REGS = 104;
    static_assert(8 * E_REGS + 4 * H_REGS + 4 * M_REGS <= 2048, "register file: 64K registers / 32 lanes");
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
        const int hslot = tid - PIPE_E_THREADS;          // ring slot of an H thread (0..127) = its tensor-memory lane
        uint32_t rKa[DW], rVa[DW];
        {   // initial fill of this thread's ring slot: registers (other side) and operand tiles (own side)
            const int key = ring_key(q0, hslot);
            if (key >= 0) {
                const uint4* ka4 = reinterpret_cast<const uint4*>(gKa + static_cast<size_t>(key) * kstep);
                const uint4* va4 = reinterpret_cast<const uint4*>(gVa + static_cast<size_t>(key) * kstep);
                const uint4* kb4 = reinterpret_cast<const uint4*>(gKb + static_cast<size_t>(key) * kstep);
                const uint4* vb4 = reinterpret_cast<const uint4*>(gVb + static_cast<size_t>(key) * kstep);
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const uint4 a = __ldg(ka4 + c), v = __ldg(va4 + c);
                    rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
                    rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
                    *reinterpret_cast<uint4*>(sKb + sw128_offset<RING>(hslot, c)) = __ldg(kb4 + c);
                    *reinterpret_cast<uint4*>(sVb + sw128_offset<RING>(hslot, c)) = __ldg(vb4 + c);
                    if (WITH_DQ) *reinterpret_cast<uint4*>(sKa + sw128_offset<RING>(hslot, c)) = a;
                }
            } else {
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    rKa[4 * c] = rKa[4 * c + 1] = rKa[4 * c + 2] = rKa[4 * c + 3] = 0;
                    rVa[4 * c] = rVa[4 * c + 1] = rVa[4 * c + 2] = rVa[4 * c + 3] = 0;
                    *reinterpret_cast<uint4*>(sKb + sw128_offset<RING>(hslot, c)) = z;
                    *reinterpret_cast<uint4*>(sVb + sw128_offset<RING>(hslot, c)) = z;
                    if (WITH_DQ) *reinterpret_cast<uint4*>(sKa + sw128_offset<RING>(hslot, c)) = z;
                }
            }
        }
        // Asynchronous staging, one commit group per call: the Q and dY rows of iteration `it`
        // (threads [0, 2*CH)) and, when next_key >= 0, the four rows of the key that enters the
        // ring with query next_key (threads [0, 4*CH)); both are waited for at the next H_sync.
        auto h_stage = [&](int it, size_t qoff, int next_key) {
            if (it >= 0 && hslot < 2 * CH) {
                const int which = hslot / CH, c = hslot % CH;
                const __nv_bfloat16* src = (which == 0 ? p.Q : p.dY) + qoff;
                const uint32_t dst = smem_u32(sStage + ((it & 1) * 2 + which) * D) + c * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                             "l"(reinterpret_cast<const uint4*>(src) + c)
                             : "memory");
            }
            if (next_key >= 0 && hslot < 4 * CH) {
                const int which = hslot / CH, c = hslot % CH;
                const __nv_bfloat16* base = which == 0 ? gKa : which == 1 ? gVa : which == 2 ? gKb : gVb;
                const uint32_t dst = smem_u32(sNext + (next_key & 1) * L::NEXT_BYTES + which * (D * 2)) + c * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                             "l"(reinterpret_cast<const uint4*>(base + static_cast<size_t>(next_key) * kstep) + c)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        h_stage(0, qoff_at(q0, 0), -1);
        fence_async_smem();
        cta_start_sync();
        constexpr int GB = L::G_BUFS;
        constexpr int HB = 8;                 // staged chunks in flight per thread (registers: 4 per chunk)
        int n = 0, it = 0, n_query = 0, ring_phase = 0;
        bool ok = true;
        float l_next = __ldg(p.l + row_at(q0, 0));
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            const bool prev_work = n > n_query;      // the previous query issued MMAs: Ring_free completes for it
            n_query = n;
            const int s = i & (RING - 1);
            uint32_t vw[4];
            ring_visibility(mask_b.row(i), i, min(p.window, x_window_oth), lane, vw);    // a pair needs a key on both axes
            const bool any_vis = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const float l_i = l_next;
                if (it + 1 < n_iter) l_next = __ldg(p.l + next_row(i, hh));
                // the staged rows of this iteration have landed; everyone is past the previous build
                asm volatile("cp.async.wait_all;" ::: "memory");
                warp_arrive(&bars[PB_H_SYNC], lane);
                ok = pipe_wait(&bars[PB_H_SYNC], it & 1, sFail);
                if (!ok) break;
                const bool boundary = hh == 0 && i > q0;      // key i replaces key i-128 in slot s
                const uint8_t* nx = sNext + (i & 1) * L::NEXT_BYTES;
                if (boundary && hslot == s) {
                    const uint4* ka4 = reinterpret_cast<const uint4*>(nx);
                    const uint4* va4 = reinterpret_cast<const uint4*>(nx + D * 2);
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        const uint4 a = ka4[c], v = va4[c];
                        rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
                        rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
                    }
                }
                if (it + 1 < n_iter) h_stage(it + 1, next_qoff(i, hh), (hh == 0 && i + 1 < q1) ? i + 1 : -1);
                const bool work = any_vis && l_i > 0.f;
                const int qb = n & 1, gb = n % GB;
                uint8_t* dQp = sQp + (x_precise ? 0 : qb) * L::TILE;      // compensated mode: buffer 0 value, buffer 1 residual
                uint8_t* dG = sG + gb * L::TILE;
                const uint4* q4 = reinterpret_cast<const uint4*>(sStage + (it & 1) * 2 * D);
                const uint4* y4 = q4 + CH;
                if (work) {
                    // Buffer reuse: Qp[n&1] was last read by the dKb MMAs of head n-2.  Each per-buffer
                    // barrier is waited on at every one of its phases.
                    if (!x_precise) { if (n >= 2) ok = pipe_wait(&bars[PB_D_DONE0 + qb], ((n >> 1) - 1) & 1, sFail); }
                    else if (n >= 1) ok = pipe_wait(&bars[PB_D_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail);
                    if (!ok) break;
                    // The staged row is read in batches of HB chunks ahead of the stores: the compiler
                    // cannot tell that the tile stores do not alias the staging area, and would otherwise
                    // run load -> multiply -> store one chunk at a time (about 100 cycles each).
#pragma unroll
                    for (int c0 = 0; c0 < CH; c0 += HB) {
                        uint4 q[HB];
#pragma unroll
                        for (int c = 0; c < HB; ++c) q[c] = q4[c0 + c];
#pragma unroll
                        for (int c = 0; c < HB; ++c) {
                            uint4 o;
                            o.x = mul_bf16x2(q[c].x, rKa[4 * (c0 + c)]);
                            o.y = mul_bf16x2(q[c].y, rKa[4 * (c0 + c) + 1]);
                            o.z = mul_bf16x2(q[c].z, rKa[4 * (c0 + c) + 2]);
                            o.w = mul_bf16x2(q[c].w, rKa[4 * (c0 + c) + 3]);
                            st_shared_v4(dQp + sw128_offset<RING>(hslot, c0 + c), o.x, o.y, o.z, o.w);
                            if (EXT && x_precise) {
                                uint4 lo;
                                lo.x = mul_residual_bf16x2(q[c].x, rKa[4 * (c0 + c)], o.x);
                                lo.y = mul_residual_bf16x2(q[c].y, rKa[4 * (c0 + c) + 1], o.y);
                                lo.z = mul_residual_bf16x2(q[c].z, rKa[4 * (c0 + c) + 2], o.z);
                                lo.w = mul_residual_bf16x2(q[c].w, rKa[4 * (c0 + c) + 3], o.w);
                                *reinterpret_cast<uint4*>(dQp + L::TILE + sw128_offset<RING>(hslot, c0 + c)) = lo;
                            }
                        }
                    }
                }
                if (boundary) {
                    // The operand-tile rows of slot s change key only after every MMA that reads the
                    // rings (and, in the dQ pass, the E warps' reads of the Kb rows) is done with the
                    // previous query; the tile built above does not depend on it, so it costs nothing.
                    if (prev_work) {
                        ok = pipe_wait(&bars[PB_RING_FREE], ring_phase & 1, sFail);
                        ++ring_phase;
                        if (!ok) break;
                    }
                    constexpr int NR = WITH_DQ ? 3 : 2;       // Kb, Vb (and Ka) rows
                    if (hslot < NR * CH) {
                        const int r = hslot / CH, c = hslot % CH;
                        const uint4 v = *reinterpret_cast<const uint4*>(nx + (r == 2 ? 0 : (2 + r)) * (D * 2) + c * 16);
                        uint8_t* tile = r == 0 ? sKb : r == 1 ? sVb : sKa;
                        *reinterpret_cast<uint4*>(tile + sw128_offset<RING>(s, c)) = v;
                    }
                }
                if (work || boundary) fence_async_smem();
                if (work) {
                    // the score product needs only this tile (and the rings)
                    warp_arrive(&bars[PB_QP_FULL0 + qb], lane);
                    // Gt[n%GB] was last read by the dVb MMAs of head n-GB
                    if (n >= GB) ok = pipe_wait(&bars[PB_V_DONE0 + gb], ((n / GB) - 1) & 1, sFail);
                    if (!ok) break;
#pragma unroll
                    for (int c0 = 0; c0 < CH; c0 += HB) {
                        uint4 y[HB];
#pragma unroll
                        for (int c = 0; c < HB; ++c) y[c] = y4[c0 + c];
#pragma unroll
                        for (int c = 0; c < HB; ++c) {
                            uint4 gq;
                            gq.x = mul_bf16x2(y[c].x, rVa[4 * (c0 + c)]);
                            gq.y = mul_bf16x2(y[c].y, rVa[4 * (c0 + c) + 1]);
                            gq.z = mul_bf16x2(y[c].z, rVa[4 * (c0 + c) + 2]);
                            gq.w = mul_bf16x2(y[c].w, rVa[4 * (c0 + c) + 3]);
                            st_shared_v4(dG + sw128_offset<RING>(hslot, c0 + c), gq.x, gq.y, gq.z, gq.w);
                        }
                    }
                    fence_async_smem();
                    warp_arrive(&bars[PB_GT_FULL0 + gb], lane);
                }
                if (work) ++n;
            }
        }
    } else if (warp >= 12) {
        reg_dec<M_REGS>();
        cta_start_sync();
        // Accumulator flushes are the work of this warpgroup: warp 12 + q reaches the tensor-memory lanes
        // of quarter q.  Quarters 1-3 belong to the three warps that otherwise only donate registers;
        // quarter 0 is flushed by the MMA warp itself, between two runs of MMAs (one query in four).
        const int fslot = (warp & 3) * 32 + lane;
        const uint32_t tlf = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        // Out of line on purpose: the 32 registers of a tensor-memory load would otherwise count
        // against the MMA warp's small budget throughout its issue loop.
        auto acc_flush = [&](int only_lane, int i_ref, bool rezero) {
            flush_acc_lanes<D>(tlf, lane, only_lane, ring_key(i_ref, fslot), gPartK, gPartV, p.scale, rezero);
        };
        const int n_bound = q1 - q0 - 1;      // query boundaries = single-lane flushes; Acc_done has one more phase
        if (!is_mma) {
            // ============================================================== flush warps (quarters 1-3)
            bool okf = true;
#pragma unroll 1
            for (int fb = 0; fb < n_bound && okf; ++fb) {
                const int i = q0 + 1 + fb, s = i & (RING - 1);
                okf = pipe_wait(&bars[PB_ACC_DONE], fb & 1, sFail);     // every MMA of the queries before i is complete
                if (okf && (warp & 3) == (s >> 5)) {
                    tc_fence_after();
                    acc_flush(s & 31, i - 1, true);
                    warp_arrive(&bars[PB_FLUSH_DONE], lane);
                }
            }
            if (okf) okf = pipe_wait(&bars[PB_ACC_DONE], n_bound & 1, sFail);
            if (okf) {
                // Drain: every slot still holds a key of (q1 - 129, q1 - 1].
                tc_fence_after();
                acc_flush(-1, q1 - 1, false);
            }
        }
        if (is_mma) {
        // ================================================================== MMA warp
        // The whole warp runs this role converged; the MMAs and commits are predicated on one
        // elected lane (see umma_ss_pred for the measured difference to a lane-0 branch).
        const uint32_t issuer = elect_one();
        const uint32_t idesc_s = make_idesc_bf16(RING, RING, 0, 0);     // score-shaped, both operands K-major
        const uint32_t idesc_acc = make_idesc_bf16(RING, D, 0, 1);      // A in TMEM, B MN-major, N = D
        // Descriptor bases are built once; a k-step only adds a compile-time constant to the
        // start-address field (16-byte units); rebuilding descriptors per MMA costs 140-190 cycles
        // an MMA against 64 cycles of tensor-pipe time.
        const uint64_t dKb = make_smem_desc(smem_u32(sKb), 16, 1024, SWIZZLE_128B);           // A, K-major
        const uint64_t dVb = make_smem_desc(smem_u32(sVb), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpK = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);          // B, K-major
        const uint64_t dGK = make_smem_desc(smem_u32(sG), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpM = make_smem_desc(smem_u32(sQp), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major
        const uint64_t dGM = make_smem_desc(smem_u32(sG), RING * 128, 1024, SWIZZLE_128B);
        const uint64_t dKaM = make_smem_desc(smem_u32(sKa), RING * 128, 1024, SWIZZLE_128B);
        const uint32_t tAK = tmem_base + C_AK, tAV = tmem_base + C_AV;
        constexpr int GB = L::G_BUFS;
        int n = 0, it = 0, n_query = 0, flushes_seen = 0;
        bool ok = true, flush_pending = false, dk_pending = false;
        (void)n_bound;
        float l_next = __ldg(p.l + row_at(q0, 0));

        // A-operand column of k-step kk inside a region: the E thread of column half c keeps its
        // BF16 results inside its own 64 score columns, P^T in the first 32 and gA^T in the last 32.
        auto a_col = [](int kk) -> uint32_t { return 64u * (kk >> 2) + 8u * (kk & 3); };
        // The MMA runs are unrolled with compile-time operand offsets (rolled loops issued ~2 % slower), and the
        // rest of this warp's code is kept compact: its instruction stream is on the critical path of every
        // hand-off, and the three roles together are close to what the instruction cache holds.  K-major
        // operands: k-step kk moves the start address (16-byte units) by 2 per step inside a 64-element
        // block and RING*8 per block.  A from tensor memory: see a_col.
        auto run_ss = [&](uint32_t tD, uint64_t dA, uint64_t dB) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                umma_ss_pred(tD, dA + off, dB + off, idesc_s, kk > 0, issuer);
            }
        };
        auto run_ts = [&](uint32_t tD, uint32_t tAop, uint64_t dB, uint32_t keep) {
#pragma unroll
            for (int kk = 0; kk < RING / 16; ++kk)
                umma_ts_pred(tD, tAop + a_col(kk), dB + kk * (2048 / 16), idesc_acc, keep | (kk > 0), issuer);
        };
        // Boundary duties.  Acc_done is committed once per boundary, after the last accumulating MMA of
        // the queries before it; the flush of the lane that changes key happens behind it, by a flush
        // warp (observed through Flush_done) or, for quarter 0, right here.
        int acc_commits = 0, self_i = 0;
        bool acc_commit_pending = false, self_pending = false;
        auto commit_acc = [&]() {
            umma_commit_pred(&bars[PB_ACC_DONE], issuer);
            ++acc_commits;
            acc_commit_pending = false;
        };
        // dKb += gA^T(m) Qp(m) for the head m = n - 1 whose gA^T the E warps finish last.
        auto issue_dk = [&](int m) {
            bool r = pipe_wait(&bars[PB_G_FULL], m & 1, sFail);
            if (r) {
                tc_fence_after();
                const uint32_t tA = tmem_base + C_R0 + (m & 1) * 128 + 32;
                const uint32_t qoff = x_precise ? 0u : (m & 1) * (L::TILE / 16);
                run_ts(tAK, tA, dQpM + qoff, 1);
                umma_commit_pred(&bars[PB_D_DONE0 + (m & 1)], issuer);
                if (acc_commit_pending) commit_acc();
            }
            return r;
        };
        auto settle_flush = [&]() {
            bool r = true;
            if (flush_pending) {
                r = pipe_wait(&bars[PB_FLUSH_DONE], flushes_seen & 1, sFail);
                ++flushes_seen;
                flush_pending = false;
                if (r) tc_fence_after();
            }
            if (r && self_pending) {
                // this warp made the commit, so it knows which phase it is waiting for
                r = pipe_wait(&bars[PB_ACC_DONE], (acc_commits - 1) & 1, sFail);
                self_pending = false;
                if (r) {
                    tc_fence_after();
                    acc_flush(self_i & 31, self_i - 1, true);
                    __syncwarp();
                    tc_fence_after();
                }
            }
            return r;
        };
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            if (i > q0) {
                // A query without work leaves its boundary unsettled: do it now, so that commits, flushes
                // and this warp's waits stay one phase apart.
                if (flush_pending || self_pending) {
                    if (dk_pending) { ok = issue_dk(n - 1); dk_pending = false; }
                    if (ok) ok = settle_flush();
                    if (!ok) break;
                }
                if (((i & (RING - 1)) >> 5) == 0) { self_pending = true; self_i = i; }
                else flush_pending = true;
                if (dk_pending) acc_commit_pending = true;   // committed right behind the kept-back dKb MMAs
                else commit_acc();
            }
            uint32_t vw[4];
            ring_visibility(mask_b.row(i), i, min(p.window, x_window_oth), lane, vw);    // a pair needs a key on both axes
            const bool any_vis = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
            bool ring_committed = false;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const float l_i = l_next;
                if (it + 1 < n_iter) l_next = __ldg(p.l + next_row(i, hh));
                if (!any_vis || !(l_i > 0.f)) {
                    // the H warps may be waiting for the kept-back MMAs before they build another tile
                    if (dk_pending) { ok = issue_dk(n - 1); dk_pending = false; }
                    continue;
                }
                const uint32_t ph = n & 1;
                const int qb = n & 1, gb = n % GB;
                const uint32_t qoff = x_precise ? 0u : qb * (L::TILE / 16), goff = gb * (L::TILE / 16);   // buffer offsets, 16-byte units
                const uint32_t tA = tmem_base + C_R0 + (n & 1) * 128;          // X^T, then P^T | gA^T
                const uint32_t tB = tmem_base + C_R0 + ((n & 1) ^ 1) * 128;    // dP^T, then W
                ok = pipe_wait(&bars[PB_QP_FULL0 + qb], (n >> 1) & 1, sFail);
                // A(n) = B(n-1): the E warps have taken dP^T (or W) of the previous head out of it
                if (ok && n > 0) ok = pipe_wait(&bars[PB_B_FREE], (n - 1) & 1, sFail);
                if (!ok) break;
                tc_fence_after();
                run_ss(tA, dKb, dQpK + qoff);                  // X^T = Kb Qp^T
                if (EXT && x_precise) {                        // + Kb (residual tile)^T
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                        umma_ss_pred(tA, dKb + off, dQpK + L::TILE / 16 + off, idesc_s, 1, issuer);
                    }
                }
                umma_commit_pred(&bars[PB_S_XT], issuer);
                if (!WITH_DQ && dk_pending) {
                    ok = issue_dk(n - 1);
                    dk_pending = false;
                    if (!ok) break;
                }
                // B(n) = A(n-1): the accumulation MMAs of the previous head read their A operand there,
                // and a later MMA is not held back for an earlier one's operand reads
                if (n > 0) ok = pipe_wait(&bars[PB_D_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail);
                if (ok) ok = pipe_wait(&bars[PB_GT_FULL0 + gb], (n / GB) & 1, sFail);
                if (!ok) break;
                tc_fence_after();
                run_ss(tB, dVb, dGK + goff);                   // dP^T = Vb Gt^T
                umma_commit_pred(&bars[PB_S_DP], issuer);
                if (!WITH_DQ && hh == G - 1) {
                    // The query's last reads of the ring tiles have been issued (without the dQ product only
                    // the two score-shaped products read them): the H warps may bring in the next key as
                    // soon as these complete, not only after the accumulation MMAs further down.
                    umma_commit_pred(&bars[PB_RING_FREE], issuer);
                    ring_committed = true;
                }
                ok = pipe_wait(&bars[PB_P_FULL], ph, sFail);
                if (ok && (flush_pending || self_pending)) ok = settle_flush();   // the lane zeroed at the query boundary
                if (!ok) break;
                tc_fence_after();
                run_ts(tAV, tA, dGM + goff, 1);                // dVb += P^T Gt
                umma_commit_pred(&bars[PB_V_DONE0 + gb], issuer);
                if (WITH_DQ) {
                    ok = pipe_wait(&bars[PB_G_FULL], ph, sFail);
                    if (!ok) break;
                    tc_fence_after();
                    // W first: the E warps wait for it, nobody is in a hurry for dKb
                    run_ts(tB, tA + 32, dKaM, 0);              // W = gA^T Ka, over the consumed dP^T columns
                    umma_commit_pred(&bars[PB_W_FULL], issuer);
                    run_ts(tAK, tA + 32, dQpM + qoff, 1);      // dKb += gA^T Qp
                    umma_commit_pred(&bars[PB_D_DONE0 + qb], issuer);
                } else if (EXT && x_precise) {
                    // both Qp buffers belong to this head: its dKb MMAs cannot be kept back behind the next head's
                    // score product, which needs the buffers rewritten first
                    ok = issue_dk(n);
                    if (!ok) break;
                } else {
                    dk_pending = true;
                }
                ++n;
            }
            // Every MMA of this query that reads the ring tiles has been issued: signal the ring rows
            // free once they complete.
            if (n > n_query && ok && !ring_committed) umma_commit_pred(&bars[PB_RING_FREE], issuer);
            n_query = n;
        }
        if (ok && dk_pending) ok = issue_dk(n - 1);
        if (ok) ok = settle_flush();
        if (ok) {
            // Final phase of Acc_done: everything has been issued; drain quarter 0 once it is complete.
            commit_acc();
            ok = pipe_wait(&bars[PB_ACC_DONE], (acc_commits - 1) & 1, sFail);
            if (ok) {
                tc_fence_after();
                acc_flush(-1, q1 - 1, false);
            }
        }
        __syncwarp();
        }
    } else {
        // ================================================================== E warps
        reg_dec<E_REGS>();
        cta_start_sync();
        const int slot = tid & (RING - 1);               // tensor-memory lane = ring slot
        const int ch = tid >> 7;                          // which 64-column half of the score tile
        const uint32_t tl = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        {   // zero both accumulators: half 0 takes dKb, half 1 dVb
            uint32_t z[32];
#pragma unroll
            for (int t = 0; t < 32; ++t) z[t] = 0;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) tmem_st32(tl + (ch ? C_AV : C_AK) + c * 32, z);
            tmem_wait_st();
            tc_fence_before();
        }
        // The accumulators must be zero before the first accumulating MMA; that MMA waits for
        // P_full of the first head, which every E warp arrives on after this point.
        // per-head scalars, fetched one iteration ahead: delta = dY . Y (from the pre-pass), m, l
        float pre_d = 0.f, pre_m = 0.f, pre_l = 0.f;
        auto prefetch = [&](size_t row) {
            pre_d = __ldg(p.delta + row);
            pre_m = __ldg(p.m + row);
            pre_l = __ldg(p.l + row);
        };
        prefetch(row_at(q0, 0));
        int n = 0, it = 0, n_query = 0;
        bool ok = true;
#pragma unroll 1
        for (int i = q0; i < q1 && ok; ++i) {
            // lanes of the score tile are own-side keys (window), columns other-side keys (window_oth)
            uint32_t vw[4], vo[4];
            ring_visibility(mask_b.row(i), i, p.window, lane, vw);
            if (x_window_oth != p.window) ring_visibility(mask_b.row(i), i, x_window_oth, lane, vo);
            else { vo[0] = vw[0]; vo[1] = vw[1]; vo[2] = vw[2]; vo[3] = vw[3]; }
            const int n_own = __popc(vw[0]) + __popc(vw[1]) + __popc(vw[2]) + __popc(vw[3]);
            const int n_oth = __popc(vo[0]) + __popc(vo[1]) + __popc(vo[2]) + __popc(vo[3]);
            const int n_vis = min(n_own, n_oth);                 // 0: no visible pair
            const bool all_vis = n_own == RING && n_oth == RING;
            const bool single = n_own * n_oth == 1;              // one visible pair: exact zero score gradients
            const bool my_vis = (vw[warp & 3] >> lane) & 1u;
            // visibility words of this thread's two 32-column chunks
            const uint32_t cw0 = my_vis ? (ch ? vo[2] : vo[0]) : 0u;
            const uint32_t cw1 = my_vis ? (ch ? vo[3] : vo[1]) : 0u;
            bool ring_arrived = false;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const size_t row = row_at(i, hh);
                const float delta = pre_d, m_i = pre_m, l_i = pre_l;
                if (it + 1 < n_iter) prefetch(next_row(i, hh));
                if (n_vis == 0 || !(l_i > 0.f)) {
                    if (WITH_DQ && tid < D) p.dQ[qoff_at(i, hh) + tid] = __float2bfloat16(0.f);
                    continue;
                }
                const float lse2 = m_i * LOG2E + __log2f(l_i);
                // packed FP32 arithmetic: one instruction for two columns
                const uint64_t c2p = pair_f32(c2, c2), lsep = pair_f32(-lse2, -lse2), dltp = pair_f32(-delta, -delta);
                const uint32_t ph = n & 1;
                const uint32_t tA = tl + C_R0 + (n & 1) * 128 + ch * 64;          // this thread's 64 score columns
                const uint32_t tB = tl + C_R0 + ((n & 1) ^ 1) * 128;
                // ---- phase 1: P^T = exp2(X^T c2 - lse) for this thread's 64 columns, BF16 into the first 32.
                // Both phases walk the columns in two rounds of 32 inside a rolled loop: half the registers
                // and half the code of one straight-line pass, and the BF16 results of a round land on
                // columns whose scores an earlier round (or this one) has already taken.
                ok = pipe_wait(&bars[PB_S_XT], ph, sFail);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t x[32], pk[16];
                    tmem_ld32(tA + cc * 32, x);
                    tmem_wait_ld();
                    const uint32_t cw = cc ? cw1 : cw0;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float a0, a1;
                        unpair_f32(fma_f32x2(pair_b32(x[t], x[t + 1]), c2p, lsep), a0, a1);
                        float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                        if (!all_vis) {
                            if (!((cw >> t) & 1u)) p0 = 0.f;
                            if (!((cw >> (t + 1)) & 1u)) p1 = 0.f;
                        }
                        pk[t >> 1] = pack_bf16x2(p0, p1);
                    }
                    tmem_st16(tA + cc * 16, pk);
                }
                tmem_wait_st();
                tc_fence_before();
                warp_arrive(&bars[PB_P_FULL], lane);
                // ---- phase 2: gA^T = P^T o (dP^T - delta), BF16 into the last 32 of this thread's columns
                ok = pipe_wait(&bars[PB_S_DP], ph, sFail);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t dp[32], pk[16];
                    tmem_ld32(tB + ch * 64 + cc * 32, dp);
                    tmem_ld16(tA + cc * 16, pk);
                    tmem_wait_ld();
                    if (!WITH_DQ && cc == 1) {
                        // dP^T is in registers: the next head's scores may land on these columns
                        tc_fence_before();
                        warp_arrive(&bars[PB_B_FREE], lane);
                    }
                    // packed BF16 product: (dP - delta) is rounded to BF16 like P before them (both are MMA
                    // operands in BF16 anyway); three instructions a pair
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float d0, d1;
                        unpair_f32(add_f32x2(pair_b32(dp[t], dp[t + 1]), dltp), d0, d1);
                        if (EXT && x_precise) {
                            // compensated mode: the product in FP32, one rounding to BF16
                            const float2 pf = unpack_bf16x2(pk[t >> 1]);
                            pk[t >> 1] = single ? 0u : pack_bf16x2(pf.x * d0, pf.y * d1);
                        } else {
                            pk[t >> 1] = single ? 0u : mul_bf16x2(pk[t >> 1], pack_bf16x2(d0, d1));
                        }
                    }
                    tmem_st16(tA + 32 + cc * 16, pk);
                }
                tmem_wait_st();
                tc_fence_before();
                warp_arrive(&bars[PB_G_FULL], lane);
                if (WITH_DQ) {
                    ok = pipe_wait(&bars[PB_W_FULL], ph, sFail);
                    if (!ok) break;
                    tc_fence_after();
                    // dQ[d] = scale * sum_k Kb_k[d] * W[k][d]; this thread: lane k, d in its half.
                    constexpr int NC = HD / 32;
                    float* red = sRed + (n & 1) * 4 * D;
#pragma unroll 1
                    for (int c = 0; c < NC; ++c) {
                        float s;
                        if (EXT && x_precise) {
                            // compensated mode: FP32 products and an FP32 lane sum
                            float va[16], vb[16];
                            {
                                uint32_t u[16];
                                tmem_ld16(tB + ch * HD + c * 32, u);
                                tmem_wait_ld();
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const uint4 kb = *reinterpret_cast<const uint4*>(
                                        sKb + sw128_offset<RING>(slot, ch * (HD / 8) + c * 4 + q));
                                    const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        const float2 kf = unpack_bf16x2(w4[e]);
                                        va[q * 8 + 2 * e] = kf.x * __uint_as_float(u[q * 8 + 2 * e]);
                                        va[q * 8 + 2 * e + 1] = kf.y * __uint_as_float(u[q * 8 + 2 * e + 1]);
                                    }
                                }
                            }
                            {
                                uint32_t u[16];
                                tmem_ld16(tB + ch * HD + c * 32 + 16, u);
                                tmem_wait_ld();
                                if (c == NC - 1) {
                                    // W is in registers: the next head's scores may land on these columns
                                    tc_fence_before();
                                    warp_arrive(&bars[PB_B_FREE], lane);
                                }
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const uint4 kb = *reinterpret_cast<const uint4*>(
                                        sKb + sw128_offset<RING>(slot, ch * (HD / 8) + c * 4 + 2 + q));
                                    const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        const float2 kf = unpack_bf16x2(w4[e]);
                                        vb[q * 8 + 2 * e] = kf.x * __uint_as_float(u[q * 8 + 2 * e]);
                                        vb[q * 8 + 2 * e + 1] = kf.y * __uint_as_float(u[q * 8 + 2 * e + 1]);
                                    }
                                }
                            }
                            // the query's last head: this warp is done with the Kb rows of the ring
                            if (c == NC - 1 && hh == G - 1) {
                                warp_arrive(&bars[PB_RING_FREE], lane);
                                ring_arrived = true;
                            }
                            s = warp_transpose_sum_2x16(va, vb, lane);
                        } else {
                            // two rounds of 16 columns keep the live set small (this role runs on 80 registers).  W is
                            // rounded to BF16 pairs and multiplied by the packed Kb words as they are: two instructions a pair
                            uint32_t w[16];
                            {
                                uint32_t u[16];
                                tmem_ld16(tB + ch * HD + c * 32, u);
                                tmem_wait_ld();
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const uint4 kb = *reinterpret_cast<const uint4*>(
                                        sKb + sw128_offset<RING>(slot, ch * (HD / 8) + c * 4 + q));
                                    const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        w[q * 4 + e] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[q * 8 + 2 * e]),
                                                                              __uint_as_float(u[q * 8 + 2 * e + 1])), w4[e]);
                                }
                            }
                            {
                                uint32_t u[16];
                                tmem_ld16(tB + ch * HD + c * 32 + 16, u);
                                tmem_wait_ld();
                                if (c == NC - 1) {
                                    // W is in registers: the next head's scores may land on these columns
                                    tc_fence_before();
                                    warp_arrive(&bars[PB_B_FREE], lane);
                                }
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const uint4 kb = *reinterpret_cast<const uint4*>(
                                        sKb + sw128_offset<RING>(slot, ch * (HD / 8) + c * 4 + 2 + q));
                                    const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        w[8 + q * 4 + e] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[q * 8 + 2 * e]),
                                                                                  __uint_as_float(u[q * 8 + 2 * e + 1])), w4[e]);
                                }
                            }
                            // the query's last head: this warp is done with the Kb rows of the ring
                            if (c == NC - 1 && hh == G - 1) {
                                warp_arrive(&bars[PB_RING_FREE], lane);
                                ring_arrived = true;
                            }
                            s = warp_transpose_sum_words(w, lane);
                        }
                        red[(warp & 3) * D + ch * HD + c * 32 + lane] = s;
                    }
                    warp_arrive(&bars[PB_E_SYNC2], lane);
                    ok = pipe_wait(&bars[PB_E_SYNC2], ph, sFail);
                    if (!ok) break;
                    if (tid < D)
                        p.dQ[qoff_at(i, hh) + tid] =
                            __float2bfloat16(p.scale * (red[tid] + red[D + tid] + red[2 * D + tid] + red[3 * D + tid]));
                }
                ++n;
            }
            // dQ pass, when the query's last head had no work: the Kb rows were last read further up
            if (WITH_DQ && ok && n > n_query && !ring_arrived) warp_arrive(&bars[PB_RING_FREE], lane);
            n_query = n;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*sFail && tid == 0) atomicExch(p.status, 3);
    if (is_mma) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Sums the partial planes of one key side into BF16 outputs.  Row k of batch b,
// KV head g was written by the query blocks that contain a query in [k, k+127]
// (clipped to [q_begin, N)); those are at most `planes` consecutive blocks, each in
// a plane of its own, so the order of the sum is fixed.
struct ReduceParams {
    const float* part_K;
    const float* part_V;
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    float* dK32;         // when non-null the sums are written here in FP32 instead (partials of a rank whose
    float* dV32;         // query heads are only a part of the KV head's: summed across ranks before rounding)
    int rows;            // B * Hkv
    int N, D, q_begin, block_len, nblk, planes;
    int bnhd, Hkv;       // layout of dK, dV (RowAddr) and KV heads per batch
    int lead;            // the writer's ring is positioned `lead` queries ahead of its first query (packed schedule: QB - 1)
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
        // a block that starts at q0 holds (and later flushes) the keys (q0 + lead - 128, ...]: row k is written by
        // the blocks that start at or before k + 127 - lead and end after k
        const int q_lo = max(k, p.q_begin), q_hi = min(k + RING - 1 - p.lead, p.N - 1);
        float4 sk = make_float4(0.f, 0.f, 0.f, 0.f), sv = sk;
        if (q_lo <= q_hi) {
            const int b_lo = (q_lo - p.q_begin) / p.block_len, b_hi = (q_hi - p.q_begin) / p.block_len;
            for (int blk = b_lo; blk <= b_hi; ++blk) {
                const size_t off = static_cast<size_t>(blk % p.planes) * plane + rk * p.D + c * 4;
                const float4 a = *reinterpret_cast<const float4*>(p.part_K + off);
                const float4 v = *reinterpret_cast<const float4*>(p.part_V + off);
                sk.x += a.x; sk.y += a.y; sk.z += a.z; sk.w += a.w;
                sv.x += v.x; sv.y += v.y; sv.z += v.z; sv.w += v.w;
            }
        }
        const size_t at = RowAddr{p.bnhd, p.Hkv, p.N, p.D}.elem(rk) + c * 4;      // the planes are [B,Hkv,N,D]; the outputs follow the layout
        if (p.dK32) {
            *reinterpret_cast<float4*>(p.dK32 + at) = sk;
            *reinterpret_cast<float4*>(p.dV32 + at) = sv;
            continue;
        }
        uint2 ok, ov;
        ok.x = pack_bf16x2(sk.x, sk.y); ok.y = pack_bf16x2(sk.z, sk.w);
        ov.x = pack_bf16x2(sv.x, sv.y); ov.y = pack_bf16x2(sv.z, sv.w);
        *reinterpret_cast<uint2*>(p.dK + at) = ok;
        *reinterpret_cast<uint2*>(p.dV + at) = ov;
    }
}

}  // namespace sgring
