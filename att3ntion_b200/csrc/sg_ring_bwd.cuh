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
//
// Schedule.  A CTA that ran these steps one after the other would spend most of its time at
// the barrier between CUDA-core and tensor-core phases, so the CTA is split into roles that
// hand work to each other through mbarriers, and every (query, head) is processed in two
// 64-column halves a/b that overlap:
//
//   H warps (4)  build the Hadamard tiles Qp = Q_i o Ka, Gt = dY_i o Va, one ring
//                row per thread; rows 0-63 (half a) and 64-127 (half b) are
//                released separately.
//   MMA warp (1) one thread issues, in order:
//                  B_a, B_b : X^T[:,x] = Kb Qp_x^T, dP^T[:,x] = Vb Gt_x^T      (N = 64)
//                  D_a, D_b : dKb += gA^T[:,x] Qp_x, dVb += P^T[:,x] Gt_x       (K = 64)
//                  W        : gA^T Ka, for dQ (dQ pass only)
//   E warps (8)  turn score columns into P^T / gA^T (BF16, back into tensor
//                memory), flush finished accumulator lanes, and collapse W to dQ.
//
// Hand-offs per processed head (all mbarriers, phase = processed-head counter):
//   H_full[x]  H -> MMA   tile half x written          D_done[x]  MMA -> H  tile half x read
//   S_full[x]  MMA -> E   score half x in TMEM          P_full[x]  E -> MMA  P^T/gA^T half x stored
//   W_full     MMA -> E   W in TMEM                     W_free     E -> MMA/H  W and the Kb rows read
// While E works on half a the tensor pipe computes half b; while the D MMAs of one
// half run, E finishes the other and H rebuilds the freed half for the next head.
// Every wait is bounded and also watches a CTA-wide failure flag, so a protocol
// error ends the kernel with a status code instead of hanging it.
#pragma once

#include "sg_ring_fwd.cuh"

namespace sgring {

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
    long long* trace;                // optional cycle counters of the pipelined schedule (null: off)
};

constexpr int PIPE_E_THREADS = 256;
constexpr int PIPE_H_THREADS = 128;
// Four full warpgroups: E (2), H (1) and one whose first warp issues the MMAs while the
// other three only hand their registers to the working roles (setmaxnreg below).
constexpr int PIPE_THREADS = PIPE_E_THREADS + PIPE_H_THREADS + 128;

template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

enum PipeBar {
    PB_H_FULL0 = 0, PB_H_FULL1, PB_S_XT, PB_S_DP, PB_P_FULL, PB_G_FULL, PB_D_DONE0, PB_D_DONE1, PB_V_DONE0, PB_V_DONE1,
    PB_W_FULL, PB_W_FREE, PB_E_SYNC, PB_E_SYNC2, PB_H_SYNC, PB_RING_FREE, PB_COUNT
};

// One arrival per warp: the lanes' earlier writes are ordered before lane 0's releasing
// arrive by the warp barrier.  256 per-thread arrivals on one barrier word serialise into
// more than a thousand cycles per hand-off; eight do not.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

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
    static constexpr int OFF_RED = OFF_STAGE + 2 * 2 * D * 2;      // 2 x 4 x D floats (dQ partials)
    static constexpr int OFF_BARS = OFF_RED + 2 * 4 * D * 4;
    static constexpr int OFF_MISC = OFF_BARS + PB_COUNT * 8;       // tmem slot (4) + fail flag (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

// Bounded wait that also leaves when another thread has raised the CTA's failure flag.
// Bounded wait on an mbarrier phase.  try_wait parks the thread in hardware until the phase
// completes or a system time limit passes.  Measured alternatives on this part, same kernel:
// all threads spinning on test_wait pulled the SM clock from 1.9 to 1.3 GHz under the power
// cap (2x the run time); one polling lane per warp with __nanosleep(20) between polls was
// 2.3x slower still (the sleep is far coarser than its argument).  The iteration count bounds
// the total wait; the loop also leaves when another thread has raised the CTA's failure flag.
__device__ __forceinline__ bool pipe_wait(uint64_t* bar, uint32_t parity, volatile int* fail,
                                          long long* trace = nullptr) {
    const uint32_t addr = smem_u32(bar);
    const long long t0 = trace ? clock64() : 0;
    for (uint32_t it = 0; it < (1u << 20); ++it) {
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
        if (done) {
            if (trace) *trace += clock64() - t0;
            return true;
        }
        if ((it & 15u) == 15u && *fail) return false;
    }
    *fail = 1;
    return false;
}

// Visibility of the 128 ring slots for query i as four ballot words; every warp
// computes the same words (lane L looks at slots L, 32+L, 64+L, 96+L).
__device__ __forceinline__ void ring_visibility(const uint8_t* mask_row, int i, int window, int lane, uint32_t (&vw)[4]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int key = ring_key(i, q * 32 + lane);
        bool v = key >= 0 && key > i - window;
        if (v && mask_row) v = mask_row[key] != 0;
        vw[q] = __ballot_sync(0xFFFFFFFFu, v);
    }
}

template <int D, bool WITH_DQ>
__global__ void __launch_bounds__(PIPE_THREADS, 1) sg_ring_bwd_kernel(const BwdParams p) {
    using L = PipeSmem<D, WITH_DQ>;
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int DW = D / 2;            // packed words per row
    constexpr int HD = D / 2;            // d columns per E thread in the dQ collapse
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t C_XT = 0, C_DP = 128, C_AK = 256, C_AV = 384;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKb = smem + L::OFF_KB;
    uint8_t* sVb = smem + L::OFF_VB;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sG = smem + L::OFF_G;
    uint8_t* sKa = smem + L::OFF_KA;
    __nv_bfloat16* sStage = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_STAGE);
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + blockIdx.x * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const int parity_buf = blockIdx.x & 1;
    const bool is_e = warp < 8, is_h = warp >= 8 && warp < 12, is_mma = warp == 12;

    (void)is_e;
    if (is_mma) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        // Arrival counts are in warps: one elected lane arrives for its warp (warp_arrive).
        mbar_init(&bars[PB_H_FULL0], 4);    mbar_init(&bars[PB_H_FULL1], 4);
        mbar_init(&bars[PB_S_XT], 1);       mbar_init(&bars[PB_S_DP], 1);
        mbar_init(&bars[PB_P_FULL], 8);     mbar_init(&bars[PB_G_FULL], 8);
        mbar_init(&bars[PB_D_DONE0], 1);    mbar_init(&bars[PB_D_DONE1], 1);
        mbar_init(&bars[PB_V_DONE0], 1);    mbar_init(&bars[PB_V_DONE1], 1);
        mbar_init(&bars[PB_W_FULL], 1);     mbar_init(&bars[PB_W_FREE], 8);
        mbar_init(&bars[PB_E_SYNC], 8);     mbar_init(&bars[PB_E_SYNC2], 8);
        mbar_init(&bars[PB_H_SYNC], 4);
        mbar_init(&bars[PB_RING_FREE], WITH_DQ ? 9 : 1);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;
    const __nv_bfloat16* gKa = p.Ka + kv_base * D;
    const __nv_bfloat16* gVa = p.Va + kv_base * D;
    const __nv_bfloat16* gKb = p.Kb + kv_base * D;
    const __nv_bfloat16* gVb = p.Vb + kv_base * D;
    float* gPartK = p.part_K + (static_cast<size_t>(parity_buf) * p.B * p.Hkv * p.N + kv_base) * D;
    float* gPartV = p.part_V + (static_cast<size_t>(parity_buf) * p.B * p.Hkv * p.N + kv_base) * D;
    const uint8_t* mask_b = p.mask ? p.mask + static_cast<size_t>(b) * p.N * p.N : nullptr;

    const int n_iter = (q1 - q0) * G;
    auto row_index = [&](int it) {
        const int i = q0 + it / G, h = g * G + it % G;
        return (static_cast<size_t>(b) * p.Hq + h) * p.N + i;
    };
    const float c2 = p.scale * LOG2E;

    // ------------------------------------------------------------------ H role state
    const int hslot = tid - PIPE_E_THREADS;          // ring slot of an H thread (0..127)
    uint32_t rKa[DW], rVa[DW];
    auto h_load_slot = [&](int key) {
        if (key >= 0) {
            const uint4* ka4 = reinterpret_cast<const uint4*>(gKa + static_cast<size_t>(key) * D);
            const uint4* va4 = reinterpret_cast<const uint4*>(gVa + static_cast<size_t>(key) * D);
            const uint4* kb4 = reinterpret_cast<const uint4*>(gKb + static_cast<size_t>(key) * D);
            const uint4* vb4 = reinterpret_cast<const uint4*>(gVb + static_cast<size_t>(key) * D);
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
    };
    auto h_stage = [&](int it) {          // H threads [0, 2*CH): one 16-byte chunk of the Q / dY row each
        if (hslot < 2 * CH) {
            const int which = hslot / CH, c = hslot % CH;
            const __nv_bfloat16* src = (which == 0 ? p.Q : p.dY) + row_index(it) * D;
            const uint32_t dst = smem_u32(sStage + ((it & 1) * 2 + which) * D) + c * 16;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                         "l"(reinterpret_cast<const uint4*>(src) + c)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Each role first sets its register budget (the CTA starts at 128 per thread: the last
    // warpgroup gives most of its registers away, the H threads take room for two ring rows,
    // the E warps keep theirs), does its share of the set-up and then meets the others at
    // one CTA barrier before the hand-off protocol starts.
    // Optional cycle accounting of the hand-off waits (one thread per role of CTA 0).
    const bool tracer = p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 &&
                        (tid == 0 || tid == PIPE_E_THREADS || tid == PIPE_E_THREADS + PIPE_H_THREADS);
    const long long t_begin = tracer ? clock64() : 0;
#define TR(k) (tracer ? p.trace + (k) : nullptr)
    // Timeline of six steady-state heads (time stamps of the hand-offs, one thread per role).
    constexpr int TL_FIRST = 804;
#define TL(ev)                                                                                          \
    do {                                                                                                \
        if (tracer && n >= TL_FIRST && n < TL_FIRST + 6)                                                \
            p.trace[32 + (WITH_DQ ? 0 : 192) + (n - TL_FIRST) * 32 + (ev)] = clock64();                 \
    } while (0)
    uint32_t tmem_base = 0;
    auto cta_start_sync = [&]() {
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        tmem_base = *tmem_slot;
    };

    if (is_h) {
        // ================================================================== H warps
        reg_inc<184>();
        h_load_slot(ring_key(q0, hslot));
        h_stage(0);
        fence_async_smem();
        cta_start_sync();
        constexpr int GB = L::G_BUFS;
        int n = 0, it = 0, n_query = 0, ring_phase = 0;
        bool ok = true;
        float l_next = __ldg(p.l + row_index(0));
        for (int i = q0; i < q1 && ok; ++i) {
            if (i > q0) {
                // Ring slot i mod 128 changes key: every MMA that reads the rings, and in the dQ
                // pass the E warps' reads of the Kb rows, must have finished with the previous
                // query.  RING_FREE completes once per query that had work, so every H thread sees
                // each of its phases in turn (a per-head barrier would be observed here only now
                // and then, and a one-bit phase parity cannot tell phases two apart).
                if (n > n_query) {
                    ok = pipe_wait(&bars[PB_RING_FREE], ring_phase & 1, sFail, TR(16));
                    ++ring_phase;
                    if (!ok) break;
                }
                if (hslot == (i & (RING - 1))) {
                    h_load_slot(i);
                    fence_async_smem();
                }
            }
            n_query = n;
            uint32_t vw[4];
            ring_visibility(mask_b ? mask_b + static_cast<size_t>(i) * p.N : nullptr, i, p.window, lane, vw);
            const bool any_vis = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const float l_i = l_next;
                if (it + 1 < n_iter) l_next = __ldg(p.l + row_index(it + 1));
                // the staged rows of this iteration have landed; everyone is past the previous build
                asm volatile("cp.async.wait_all;" ::: "memory");
                warp_arrive(&bars[PB_H_SYNC], lane);
                ok = pipe_wait(&bars[PB_H_SYNC], it & 1, sFail, TR(17));
                if (!ok) break;
                TL(20);
                if (it + 1 < n_iter) h_stage(it + 1);
                if (!any_vis || !(l_i > 0.f)) continue;
                // Buffer reuse: Qp[n&1] was last read by the dKb MMAs of head n-2, Gt[n%GB] by the dVb
                // MMAs of head n-GB.  Each per-buffer barrier is waited on at every one of its phases.
                const int qb = n & 1, gb = n % GB;
                if (n >= 2) ok = pipe_wait(&bars[PB_D_DONE0 + qb], ((n >> 1) - 1) & 1, sFail, TR(18));
                if (ok && n >= GB) ok = pipe_wait(&bars[PB_V_DONE0 + gb], ((n / GB) - 1) & 1, sFail, TR(18));
                if (!ok) break;
                TL(21);
                uint8_t* dQp = sQp + qb * L::TILE;
                uint8_t* dG = sG + gb * L::TILE;
                const long long th0 = tracer ? clock64() : 0;
                const uint4* q4 = reinterpret_cast<const uint4*>(sStage + (it & 1) * 2 * D);
                const uint4* y4 = q4 + CH;
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const uint4 q = q4[c], y = y4[c];
                    uint4 o, gq;
                    o.x = mul_bf16x2(q.x, rKa[4 * c]);      gq.x = mul_bf16x2(y.x, rVa[4 * c]);
                    o.y = mul_bf16x2(q.y, rKa[4 * c + 1]);  gq.y = mul_bf16x2(y.y, rVa[4 * c + 1]);
                    o.z = mul_bf16x2(q.z, rKa[4 * c + 2]);  gq.z = mul_bf16x2(y.z, rVa[4 * c + 2]);
                    o.w = mul_bf16x2(q.w, rKa[4 * c + 3]);  gq.w = mul_bf16x2(y.w, rVa[4 * c + 3]);
                    *reinterpret_cast<uint4*>(dQp + sw128_offset<RING>(hslot, c)) = o;
                    *reinterpret_cast<uint4*>(dG + sw128_offset<RING>(hslot, c)) = gq;
                }
                const long long th1 = tracer ? clock64() : 0;
                fence_async_smem();
                warp_arrive(&bars[PB_H_FULL0 + qb], lane);
                if (tracer) { p.trace[24] += th1 - th0; p.trace[25] += clock64() - th1; }
                TL(22);
                ++n;
            }
        }
    } else if (warp >= 12) {
        reg_dec<72>();
        cta_start_sync();
        if (is_mma) {
        // ================================================================== MMA warp
        const uint32_t idesc_s = make_idesc_bf16(RING, RING, 0, 0);     // score-shaped, both operands K-major
        const uint32_t idesc_acc = make_idesc_bf16(RING, D, 0, 1);      // A in TMEM, B MN-major, N = D
        // Descriptor bases are built once; a k-step only adds a compile-time constant to the
        // start-address field (16-byte units).  Measured on one CTA (128x128x16 MMAs, 64 cycles
        // of tensor-pipe time each): one thread issuing an unrolled run with precomputed
        // descriptors sustains 64 cycles an MMA; electing a lane per MMA costs 102, and
        // rebuilding descriptors per MMA 140-190.
        const uint64_t dKb = make_smem_desc(smem_u32(sKb), 16, 1024, SWIZZLE_128B);           // A, K-major
        const uint64_t dVb = make_smem_desc(smem_u32(sVb), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpK = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);          // B, K-major
        const uint64_t dGK = make_smem_desc(smem_u32(sG), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpM = make_smem_desc(smem_u32(sQp), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major
        const uint64_t dGM = make_smem_desc(smem_u32(sG), RING * 128, 1024, SWIZZLE_128B);
        const uint64_t dKaM = make_smem_desc(smem_u32(sKa), RING * 128, 1024, SWIZZLE_128B);
        const uint32_t tXT = tmem_base + C_XT, tDP = tmem_base + C_DP, tAK = tmem_base + C_AK, tAV = tmem_base + C_AV;
        int n = 0, it = 0, n_query = 0;
        bool ok = true;
        float l_next = __ldg(p.l + row_index(0));
        for (int i = q0; i < q1 && ok; ++i) {
            uint32_t vw[4];
            ring_visibility(mask_b ? mask_b + static_cast<size_t>(i) * p.N : nullptr, i, p.window, lane, vw);
            const bool any_vis = (vw[0] | vw[1] | vw[2] | vw[3]) != 0;
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const float l_i = l_next;
                if (it + 1 < n_iter) l_next = __ldg(p.l + row_index(it + 1));
                if (!any_vis || !(l_i > 0.f)) continue;
                {   // the warp waits together; lane 0 issues each operand's MMAs back to back and commits them
                    const uint32_t ph = n & 1;
                    // The score MMAs overwrite the tensor-memory columns that the previous head's
                    // accumulation and W MMAs read their A operand from; a later MMA is not held back
                    // for an earlier one's operand reads, so wait for the previous head's last group.
                    constexpr int GB = L::G_BUFS;
                    const int qb = n & 1, gb = n % GB;
                    const uint32_t qoff = qb * (L::TILE / 16), goff = gb * (L::TILE / 16);   // buffer offsets, 16-byte units
                    if (n > 0)
                        ok = WITH_DQ ? pipe_wait(&bars[PB_W_FULL], (n - 1) & 1, sFail, TR(0))
                                     : pipe_wait(&bars[PB_D_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, TR(0));
                    TL(0);
                    if (ok) ok = pipe_wait(&bars[PB_H_FULL0 + qb], (n >> 1) & 1, sFail, TR(1));
                    TL(1);
                    if (ok) {
                        tc_fence_after();
                        if (lane == 0) {
#pragma unroll
                            for (int kk = 0; kk < D / 16; ++kk) {      // X^T = Kb Qp^T
                                const uint32_t off = ((kk >> 2) * (RING * 128) + (kk & 3) * 32) / 16;
                                umma_ss(tXT, dKb + off, dQpK + (off + qoff), idesc_s, kk > 0);
                            }
                            umma_commit(&bars[PB_S_XT]);
                        }
                        __syncwarp();
                        // dP^T lands on the columns that held W of the previous head
                        TL(2);
                        if (WITH_DQ && n > 0) ok = pipe_wait(&bars[PB_W_FREE], (n - 1) & 1, sFail, TR(3));
                        TL(3);
                    }
                    if (ok) {
                        if (lane == 0) {
#pragma unroll
                            for (int kk = 0; kk < D / 16; ++kk) {      // dP^T = Vb Gt^T
                                const uint32_t off = ((kk >> 2) * (RING * 128) + (kk & 3) * 32) / 16;
                                umma_ss(tDP, dVb + off, dGK + (off + goff), idesc_s, kk > 0);
                            }
                            umma_commit(&bars[PB_S_DP]);
                        }
                        __syncwarp();
                        TL(4);
                        ok = pipe_wait(&bars[PB_P_FULL], ph, sFail, TR(4));
                        TL(5);
                    }
                    if (ok) {
                        tc_fence_after();
                        if (lane == 0) {
#pragma unroll
                            for (int kk = 0; kk < RING / 16; ++kk)    // dVb += P^T Gt
                                umma_ts(tAV, tXT + kk * 8, dGM + (kk * (2048 / 16) + goff), idesc_acc, 1);
                            umma_commit(&bars[PB_V_DONE0 + gb]);
                        }
                        __syncwarp();
                        TL(6);
                        ok = pipe_wait(&bars[PB_G_FULL], ph, sFail, TR(5));
                        TL(7);
                    }
                    if (ok) {
                        tc_fence_after();
                        if (lane == 0) {
#pragma unroll
                            for (int kk = 0; kk < RING / 16; ++kk)    // dKb += gA^T Qp
                                umma_ts(tAK, tXT + 64 + kk * 8, dQpM + (kk * (2048 / 16) + qoff), idesc_acc, 1);
                            umma_commit(&bars[PB_D_DONE0 + qb]);
                            if (WITH_DQ) {
#pragma unroll
                                for (int kk = 0; kk < RING / 16; ++kk)    // W = gA^T Ka, over the consumed dP^T columns
                                    umma_ts(tDP, tXT + 64 + kk * 8, dKaM + kk * (2048 / 16), idesc_acc, kk > 0);
                                umma_commit(&bars[PB_W_FULL]);
                            }
                        }
                        __syncwarp();
                        TL(8);
                    }
                }
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
                ++n;
            }
            // every MMA of this query has been issued: signal the ring rows free once they complete
            if (n > n_query && ok && lane == 0) umma_commit(&bars[PB_RING_FREE]);
            __syncwarp();
            n_query = n;
        }
        // Let the last committed group finish before the tensor memory is released.
        if (n > 0 && ok) {
            if (WITH_DQ) pipe_wait(&bars[PB_W_FULL], (n - 1) & 1, sFail);
            else pipe_wait(&bars[PB_D_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail);
        }
        __syncwarp();
        }
    } else {
        // ================================================================== E warps
        cta_start_sync();
        const int slot = tid & (RING - 1);               // tensor-memory lane = ring slot
        const int ch = tid >> 7;                          // which 32-column chunk of each half
        const uint32_t tl = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        {
            uint32_t z[32];
#pragma unroll
            for (int t = 0; t < 32; ++t) z[t] = 0;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) tmem_st32(tl + (ch ? C_AV : C_AK) + c * 32, z);
            tmem_wait_st();
            tc_fence_before();
        }
        auto flush = [&](int quarter, int only_lane, int i_ref, bool rezero) {
            if ((warp & 3) != quarter) return;
            const uint32_t col = ch ? C_AV : C_AK;
            float* dst_base = ch ? gPartV : gPartK;
            const float mul = ch ? 1.0f : p.scale;
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
            if (rezero) {
                tmem_wait_st();
                tc_fence_before();
            }
        };
        // per-head scalars, fetched one iteration ahead: this lane's slice of dY and Y, and m, l
        uint2 pre_dy = make_uint2(0, 0), pre_y = make_uint2(0, 0);
        uint32_t pre_dy2[2] = {0, 0}, pre_y2[2] = {0, 0};
        float pre_m = 0.f, pre_l = 0.f;
        auto prefetch = [&](int it) {
            const size_t row = row_index(it);
            if (D == 128) {
                pre_dy = __ldg(reinterpret_cast<const uint2*>(p.dY + row * D) + lane);
                pre_y = __ldg(reinterpret_cast<const uint2*>(p.Y + row * D) + lane);
            } else {
                pre_dy2[0] = __ldg(reinterpret_cast<const uint32_t*>(p.dY + row * D) + lane);
                pre_y2[0] = __ldg(reinterpret_cast<const uint32_t*>(p.Y + row * D) + lane);
            }
            pre_m = __ldg(p.m + row);
            pre_l = __ldg(p.l + row);
        };
        prefetch(0);
        // last MMA group of head k: W (dQ pass, one barrier, phase k) or dKb (per-buffer barrier, phase k/2)
        auto wait_head_done = [&](int k, long long* tr) {
            return WITH_DQ ? pipe_wait(&bars[PB_W_FULL], k & 1, sFail, tr)
                           : pipe_wait(&bars[PB_D_DONE0 + (k & 1)], (k >> 1) & 1, sFail, tr);
        };
        int n = 0, it = 0, n_query = 0;
        bool ok = true;
        for (int i = q0; i < q1 && ok; ++i) {
            if (i > q0) {
                if (n > 0) {
                    ok = wait_head_done(n - 1, TR(13));
                    if (!ok) break;
                    tc_fence_after();
                }
                const int s = i & (RING - 1);
                flush(s >> 5, s & 31, i - 1, true);
            }
            uint32_t vw[4];
            ring_visibility(mask_b ? mask_b + static_cast<size_t>(i) * p.N : nullptr, i, p.window, lane, vw);
            const int n_vis = __popc(vw[0]) + __popc(vw[1]) + __popc(vw[2]) + __popc(vw[3]);
            const bool all_vis = n_vis == RING;
            const bool single = n_vis == 1;
            const bool my_vis = (vw[warp & 3] >> lane) & 1u;
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const size_t row = row_index(it);
                // delta = dY . Y and lse (log2 units) of this head from the prefetched slices
                float delta;
                if (D == 128) {
                    const float2 a0 = unpack_bf16x2(pre_dy.x), a1 = unpack_bf16x2(pre_dy.y);
                    const float2 b0 = unpack_bf16x2(pre_y.x), b1 = unpack_bf16x2(pre_y.y);
                    delta = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
                } else {
                    const float2 a0 = unpack_bf16x2(pre_dy2[0]), b0 = unpack_bf16x2(pre_y2[0]);
                    delta = a0.x * b0.x + a0.y * b0.y;
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) delta += __shfl_xor_sync(0xFFFFFFFFu, delta, o);
                const float m_i = pre_m, l_i = pre_l;
                if (it + 1 < n_iter) prefetch(it + 1);
                if (n_vis == 0 || !(l_i > 0.f)) {
                    if (WITH_DQ && tid < D) p.dQ[row * D + tid] = __float2bfloat16(0.f);
                    continue;
                }
                const float lse2 = m_i * LOG2E + __log2f(l_i);
                const uint32_t ph = n & 1;
                // ---- phase 1: P^T = exp2(X^T c - lse) for this thread's 64 columns, BF16 into X^T[0,64)
                uint32_t pk[32];
                TL(10);
                ok = pipe_wait(&bars[PB_S_XT], ph, sFail, TR(8));
                if (!ok) break;
                TL(11);
                tc_fence_after();
                long long tt = tracer ? clock64() : 0;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int c = 2 * ch + cc;                      // 32-column chunk of the score tile
                    uint32_t xr[32];
                    tmem_ld32(tl + C_XT + c * 32, xr);
                    tmem_wait_ld();
                    const uint32_t cw = my_vis ? (c == 0 ? vw[0] : c == 1 ? vw[1] : c == 2 ? vw[2] : vw[3]) : 0u;
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(xr[t]), c2, -lse2));
                        float p1 = fast_exp2(fmaf(__uint_as_float(xr[t + 1]), c2, -lse2));
                        if (!all_vis) {
                            if (!((cw >> t) & 1u)) p0 = 0.f;
                            if (!((cw >> (t + 1)) & 1u)) p1 = 0.f;
                        }
                        pk[cc * 16 + (t >> 1)] = pack_bf16x2(p0, p1);
                    }
                }
                if (tracer) { const long long t2 = clock64(); p.trace[21] += t2 - tt; tt = t2; }
                // the BF16 results land on score columns that other E threads read: all loads first
                tc_fence_before();
                TL(12);
                warp_arrive(&bars[PB_E_SYNC], lane);
                ok = pipe_wait(&bars[PB_E_SYNC], ph, sFail, TR(10));
                if (!ok) break;
                TL(13);
                tc_fence_after();
                tmem_st32(tl + C_XT + ch * 32, pk);
                tmem_wait_st();
                tc_fence_before();
                warp_arrive(&bars[PB_P_FULL], lane);
                TL(14);
                // ---- phase 2: gA^T = P^T o (dP^T - delta), BF16 into X^T[64,128)
                ok = pipe_wait(&bars[PB_S_DP], ph, sFail, TR(9));
                if (!ok) break;
                TL(15);
                tc_fence_after();
                if (tracer) tt = clock64();
                {
                    uint32_t gk[32];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t dp[32];
                        tmem_ld32(tl + C_DP + (2 * ch + cc) * 32, dp);
                        tmem_wait_ld();
#pragma unroll
                        for (int t = 0; t < 32; t += 2) {
                            const float2 pp = unpack_bf16x2(pk[cc * 16 + (t >> 1)]);
                            float g0 = pp.x * (__uint_as_float(dp[t]) - delta);
                            float g1 = pp.y * (__uint_as_float(dp[t + 1]) - delta);
                            if (single) { g0 = 0.f; g1 = 0.f; }
                            gk[cc * 16 + (t >> 1)] = pack_bf16x2(g0, g1);
                        }
                    }
                    tmem_st32(tl + C_XT + 64 + ch * 32, gk);
                    tmem_wait_st();
                    tc_fence_before();
                }
                if (tracer) p.trace[22] += clock64() - tt;
                warp_arrive(&bars[PB_G_FULL], lane);
                TL(16);
                if (!ok) break;
                if (WITH_DQ) {
                    ok = pipe_wait(&bars[PB_W_FULL], ph, sFail, TR(11));
                    if (!ok) break;
                    TL(17);
                    tc_fence_after();
                    const long long te = tracer ? clock64() : 0;
                    // dQ[d] = scale * sum_k Kb_k[d] * W[k][d]; this thread: lane k, d in its half.
                    const uint32_t wcol = C_DP + ch * HD;
                    constexpr int NC = HD / 32;
                    float* red = sRed + (n & 1) * 4 * D;
#pragma unroll 1
                    for (int c = 0; c < NC; ++c) {
                        uint32_t u[32];
                        float v[32];
                        tmem_ld32(tl + wcol + c * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 kb = *reinterpret_cast<const uint4*>(
                                sKb + sw128_offset<RING>(slot, ch * (HD / 8) + c * 4 + q));
                            const uint32_t w4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 kf = unpack_bf16x2(w4[e]);
                                v[q * 8 + 2 * e] = kf.x * __uint_as_float(u[q * 8 + 2 * e]);
                                v[q * 8 + 2 * e + 1] = kf.y * __uint_as_float(u[q * 8 + 2 * e + 1]);
                            }
                        }
                        if (c == NC - 1) {
                            // W and this thread's Kb row are in registers: the next head may overwrite them
                            tc_fence_before();
                            warp_arrive(&bars[PB_W_FREE], lane);
                        }
                        const float s = warp_transpose_sum(v, lane);
                        red[(warp & 3) * D + ch * HD + c * 32 + lane] = s;
                    }
                    if (tracer) p.trace[23] += clock64() - te;
                    TL(18);
                    warp_arrive(&bars[PB_E_SYNC2], lane);
                    ok = pipe_wait(&bars[PB_E_SYNC2], ph, sFail, TR(12));
                    if (!ok) break;
                    TL(19);
                    if (tid < D)
                        p.dQ[row * D + tid] =
                            __float2bfloat16(p.scale * (red[tid] + red[D + tid] + red[2 * D + tid] + red[3 * D + tid]));
                }
                ++n;
            }
            // dQ pass: this warp has read the Kb rows of the query's last head (in its epilogue)
            if (WITH_DQ && ok && n > n_query) warp_arrive(&bars[PB_RING_FREE], lane);
            n_query = n;
        }
        // Drain: every slot still holds a key of (q1 - 129, q1 - 1].
        if (ok) {
            if (n > 0) {
                ok = wait_head_done(n - 1, nullptr);
                tc_fence_after();
            }
            if (ok) {
#pragma unroll 1
                for (int quarter = 0; quarter < 4; ++quarter) flush(quarter, -1, q1 - 1, false);
            }
        }
    }
    if (tracer) p.trace[tid == 0 ? 14 : (tid == PIPE_E_THREADS ? 19 : 6)] += clock64() - t_begin;
#undef TR
#undef TL
    tc_fence_before();
    __syncthreads();
    if (*sFail && tid == 0) atomicExch(p.status, 3);
    if (is_mma) tmem_dealloc(tmem_base, TMEM_COLS);
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
