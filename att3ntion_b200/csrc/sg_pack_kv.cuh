// Key-side gradients of the windowed single gather for windows of at most 64 keys ("packed" schedule), sm_100a.
//
// One launch yields the gradients of one key side, as sg_ring_bwd.cuh does (two launches with the sides
// exchanged; reference: cuda/backward.cu:415-934 with ROLE = BWD_QUERY_ROWS, small-window schedules in
// cuda/shared_kv/shared_retained_rs.cuh:280-2470).  With the own side called (Kb, Vb) and the other (Ka, Va):
//
//   dKb[k] = scale * sum_{i,h,j} gA[j][k] (Q_i o Ka_j)        dVb[k] = sum_{i,h,j} P[j][k] (dY_i o Va_j)
//
// The own keys keep the 128-slot ring of sg_ring_bwd.cuh: key k in slot k mod 128 of the operand tiles and in
// lane k mod 128 of two FP32 accumulators in tensor memory that persist across the queries and heads a CTA
// walks.  What changes is the other side of the score tile.  A window of W <= 64 keys fills only W of its 128
// columns, so QB = 128 / W consecutive queries share a tile, exactly as in sg_pack_q.cuh:
//
//   tile column (g, js), g < QB, js < W:  query i0 + g, other-side key ring_key_w(i0 + g, js)
//   tile lane ks < 128:                   own-side key ring_key(i0 + QB - 1, ks)
//
// The two Hadamard tiles have one row per column, (Q_{i0+g} o Ka) and (dY_{i0+g} o Va); the accumulating
// products contract over all 128 columns at once, i.e. over the QB queries and their keys together, which is
// the sum the gradients need.  P^T and gA^T are elementwise with per-column-group constants (the forward's
// statistics and delta = dY.Y of the column's query, the latter precomputed by a small kernel).  dQ does not
// come out of this orientation; sg_pack_q.cuh produces it.
//
// Roles, tensor-memory regions and hand-offs are those of sg_ring_bwd.cuh without its dQ branch; a "query
// boundary" there is a tile boundary here (QB keys enter, QB accumulator lanes are flushed).
#pragma once

#include "sg_pack_q.cuh"
#include "sg_ring_bwd.cuh"

namespace sgpack {

struct KvParams {
    const __nv_bfloat16* Q;          // [B,Hq,N,D]
    const __nv_bfloat16* dY;         // [B,Hq,N,D]
    const float* m;                  // [B,Hq,N]
    const float* l;
    const float* delta;              // [B,Hq,N]  rowsum(dY o Y)
    const __nv_bfloat16* Ka;         // other key side   [B,Hkv,N,D]
    const __nv_bfloat16* Va;
    const __nv_bfloat16* Kb;         // own key side: gradients are produced for these
    const __nv_bfloat16* Vb;
    const uint8_t* mask;             // [B,N,N] or null
    const uint32_t* mask_words;    // the same mask as packed words [B,N,ceil(N/32)], or null (takes precedence)
    float* part_K;                   // [planes][B,Hkv,N,D] FP32 partials of dKb (plane-major)
    float* part_V;
    int B, Hq, Hkv, N, window, q_begin, block_len, planes;
    int bnhd;                        // memory layout of Q, dY and the key tensors: 0 [B,H,N,D], 1 [B,N,H,D] (RowAddr)
    float scale;
    int* status;
};

enum KvBar {
    KB_QP_FULL0 = 0, KB_QP_FULL1, KB_GT_FULL0, KB_GT_FULL1, KB_S_XT, KB_S_DP, KB_P_FULL, KB_G_FULL, KB_D_DONE0, KB_D_DONE1,
    KB_V_DONE0, KB_V_DONE1, KB_B_FREE, KB_H_SYNC, KB_RING_FREE, KB_FLUSH_DONE, KB_ACC_DONE, KB_COUNT
};

template <int D, int W>
struct KvSmem {
    static constexpr int QBN = RING / W;
    static constexpr int TILE = RING * D * 2;
    static constexpr int OFF_KB = 0;
    static constexpr int OFF_VB = TILE;
    static constexpr int OFF_QP = 2 * TILE;                        // 2 buffers
    static constexpr int OFF_G = 4 * TILE;                         // 2 buffers
    static constexpr int OFF_STAGE = 6 * TILE;                     // 2 stages x {Q, dY} x QBN rows
    static constexpr int STAGE_BYTES = 2 * QBN * D * 2;
    static constexpr int NEXT_BYTES = 4 * QBN * D * 2;             // rows Ka, Va, Kb, Vb of the QBN keys of one tile
    static constexpr int OFF_NEXT = OFF_STAGE + 2 * STAGE_BYTES;   // 2 buffers (tile parity)
    static constexpr int OFF_BARS = OFF_NEXT + 2 * NEXT_BYTES;
    static constexpr int OFF_MISC = OFF_BARS + KB_COUNT * 8;       // tmem slot (4) + fail flag (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

// delta[row] = sum_d dY[row][d] * Y[row][d] in FP32, one warp per row (the reference's delta128,
// cuda/shared_kv/shared_delta.cuh:9-29).
template <int D>
__global__ void sg_delta_kernel(const __nv_bfloat16* dY, const __nv_bfloat16* Y, float* delta, size_t rows, int bnhd,
                                int H, int N) {
    const size_t srow = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;    // [B,H,N] index
    const int lane = threadIdx.x & 31;
    if (srow >= rows) return;
    const size_t row = RowAddr{bnhd, H, N, D}.elem(srow) / D;
    float acc = 0.f;
    constexpr int PER_LANE = D / 32;        // 4 (D = 128) or 2 (D = 64) elements
    if (PER_LANE == 4) {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(dY + row * D) + lane);
        const uint2 y = __ldg(reinterpret_cast<const uint2*>(Y + row * D) + lane);
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y);
        acc = a0.x * y0.x + a0.y * y0.y + a1.x * y1.x + a1.y * y1.y;
    } else {
        const uint32_t a = __ldg(reinterpret_cast<const uint32_t*>(dY + row * D) + lane);
        const uint32_t y = __ldg(reinterpret_cast<const uint32_t*>(Y + row * D) + lane);
        const float2 a0 = unpack_bf16x2(a), y0 = unpack_bf16x2(y);
        acc = a0.x * y0.x + a0.y * y0.y;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) delta[srow] = acc;
}

// Copies the accumulator lanes [lane_lo, lane_lo + count) of a warp's quarter (count < 0: all 32) to the FP32
// partial planes and, on request, zeroes them.  `key` is the key of this thread's lane (< 0: none).
template <int D>
__device__ __noinline__ void flush_acc_range(uint32_t tl, int lane, int lane_lo, int count, int key, float* part_k,
                                             float* part_v, float scale, bool rezero) {
    constexpr uint32_t C_AK = 256, C_AV = 384;
    const bool sel = count < 0 || (lane >= lane_lo && lane < lane_lo + count);
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

template <int D, int W>
__global__ void __launch_bounds__(PIPE_THREADS, 1) sg_pack_kv_kernel(const KvParams p) {
    using L = KvSmem<D, W>;
    constexpr int QBN = RING / W;
    constexpr int CH = D / 8;
    constexpr int DW = D / 2;
    constexpr int NG = 64 / W > 0 ? 64 / W : 1;      // column groups (queries) per 64-column half: 4, 2, 1
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t C_R0 = 0, C_AK = 256, C_AV = 384;   // R1 = R0 + 128
    static_assert(D == 128, "packed schedule: D = 128 only");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKb = smem + L::OFF_KB;
    uint8_t* sVb = smem + L::OFF_VB;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sG = smem + L::OFF_G;
    uint8_t* sStage = smem + L::OFF_STAGE;
    uint8_t* sNext = smem + L::OFF_NEXT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y, bx = blockIdx.x;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + bx * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const int n_tiles = (q1 - q0) / QBN;
    const int plane_idx = bx % p.planes;
    const bool is_h = warp >= 8 && warp < 12, is_mma = warp == 12;

    if (is_mma) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&bars[KB_QP_FULL0], 4);   mbar_init(&bars[KB_QP_FULL1], 4);
        mbar_init(&bars[KB_GT_FULL0], 4);   mbar_init(&bars[KB_GT_FULL1], 4);
        mbar_init(&bars[KB_S_XT], 1);       mbar_init(&bars[KB_S_DP], 1);
        mbar_init(&bars[KB_P_FULL], 8);     mbar_init(&bars[KB_G_FULL], 8);
        mbar_init(&bars[KB_D_DONE0], 1);    mbar_init(&bars[KB_D_DONE1], 1);
        mbar_init(&bars[KB_V_DONE0], 1);    mbar_init(&bars[KB_V_DONE1], 1);
        mbar_init(&bars[KB_B_FREE], 8);     mbar_init(&bars[KB_H_SYNC], 4);
        mbar_init(&bars[KB_RING_FREE], 1);
        mbar_init(&bars[KB_FLUSH_DONE], 1); mbar_init(&bars[KB_ACC_DONE], 1);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;       // statistics-style row index of key 0
    const RowAddr kaddr{p.bnhd, p.Hkv, p.N, D};
    const size_t kstep = kaddr.step();                                       // elements from one key's row to the next
    const __nv_bfloat16* gKa = p.Ka + kaddr.elem(kv_base);
    const __nv_bfloat16* gVa = p.Va + kaddr.elem(kv_base);
    const __nv_bfloat16* gKb = p.Kb + kaddr.elem(kv_base);
    const __nv_bfloat16* gVb = p.Vb + kaddr.elem(kv_base);
    float* gPartK = p.part_K + (static_cast<size_t>(plane_idx) * p.B * p.Hkv * p.N + kv_base) * D;
    float* gPartV = p.part_V + (static_cast<size_t>(plane_idx) * p.B * p.Hkv * p.N + kv_base) * D;
    const MaskView mask_b = mask_view(p.mask, p.mask_words, b, p.N);
    const int n_iter = n_tiles * G;
    auto row_at = [&](int i, int hh) {
        return (static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i;
    };
    // Element offset of the row of (position i, head hh of this KV group) in Q, dY, Y, dQ, its tensor-map coordinates,
    // and the coordinates of a key's row (RowAddr describes the two layouts; here without its divisions).
    auto qoff_at = [&](int i, int hh) -> size_t {
        return p.bnhd ? ((static_cast<size_t>(b) * p.N + i) * p.Hq + (g * G + hh)) * D
                      : ((static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i) * D;
    };
    auto q_tma = [&](int i, int hh, int& x, int& y) {
        if (p.bnhd) { x = (g * G + hh) * D; y = b * p.N + i; }
        else { x = 0; y = (b * p.Hq + (g * G + hh)) * p.N + i; }
    };
    auto k_tma = [&](int key, int& x, int& y) {
        if (p.bnhd) { x = g * D; y = b * p.N + key; }
        else { x = 0; y = static_cast<int>(kv_base) + key; }
    };
    const size_t qstep = p.bnhd ? static_cast<size_t>(p.Hq) * D : D;      // elements between consecutive positions of one head
    const float c2 = p.scale * LOG2E;

    auto tile_has_work = [&](int i0) {
        if (!mask_b.any()) return true;
        uint32_t any = 0;
#pragma unroll 1
        for (int gg = 0; gg < QBN; ++gg) {
            uint32_t vw[4];
            column_visibility(mask_b.row(i0 + gg), i0 + gg, i0 + QBN - 1, p.window, lane, vw);
            any |= vw[0] | vw[1] | vw[2] | vw[3];
        }
        return any != 0;
    };

    constexpr int E_REGS = 88, H_REGS = 232, M_REGS = 104;
    static_assert(8 * E_REGS + 4 * H_REGS + 4 * M_REGS <= 2048, "register file: 64K registers / 32 lanes");
    uint32_t tmem_base = 0;
    auto cta_start_sync = [&]() {
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        tmem_base = *tmem_slot;
    };
    // rows of the keys of tile `t` in the staging buffers: plane 0 Ka, 1 Va, 2 Kb, 3 Vb
    auto next_row = [&](int plane, int key) {
        const int t = (key - q0) / QBN;
        return sNext + (t & 1) * L::NEXT_BYTES + (plane * QBN + (key - q0) % QBN) * (D * 2);
    };

    if (is_h) {
        // ================================================================== H warps
        reg_inc<H_REGS>();
        const int hslot = tid - PIPE_E_THREADS;          // tile column of this thread = row of the Hadamard tiles
        const int hg = hslot / W, hjs = hslot & (W - 1);
        uint32_t rKa[DW], rVa[DW];
        int kcur = ring_key_w<W>(q0 + hg, hjs);
        {   // initial fill: own-side ring rows (slot = this thread's index), this column's other-side rows,
            // and the first tile's keys in the staging buffer the next tile's columns are refreshed from
            const int okey = ring_key(q0 + QBN - 1, hslot);
            const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                uint4 kb = z, vb = z, a = z, v = z;
                if (okey >= 0) {
                    kb = __ldg(reinterpret_cast<const uint4*>(gKb + static_cast<size_t>(okey) * kstep) + c);
                    vb = __ldg(reinterpret_cast<const uint4*>(gVb + static_cast<size_t>(okey) * kstep) + c);
                }
                if (kcur >= 0) {
                    a = __ldg(reinterpret_cast<const uint4*>(gKa + static_cast<size_t>(kcur) * kstep) + c);
                    v = __ldg(reinterpret_cast<const uint4*>(gVa + static_cast<size_t>(kcur) * kstep) + c);
                }
                *reinterpret_cast<uint4*>(sKb + sw128_offset<RING>(hslot, c)) = kb;
                *reinterpret_cast<uint4*>(sVb + sw128_offset<RING>(hslot, c)) = vb;
                rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
                rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
            }
            for (int x = hslot; x < 2 * QBN * CH; x += PIPE_H_THREADS) {      // other-side rows of tile 0's keys
                const int plane = x / (QBN * CH), rem = x % (QBN * CH), kr = rem / CH, c = rem % CH;
                const __nv_bfloat16* base = plane == 0 ? gKa : gVa;
                *reinterpret_cast<uint4*>(next_row(plane, q0 + kr) + c * 16) =
                    __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(q0 + kr) * kstep) + c);
            }
        }
        // Asynchronous staging, one commit group per call: the QBN Q and dY rows of iteration `it` and, when
        // next_tile > 0, the four rows of each key that enters with that tile; both are waited for at the next H_sync.
        auto h_stage = [&](int it, size_t qoff, int next_tile) {
            if (it >= 0) {
                for (int x = hslot; x < 2 * QBN * CH; x += PIPE_H_THREADS) {
                    const int which = x / (QBN * CH), rem = x % (QBN * CH);
                    // the rows of QBN consecutive queries of one head: qstep elements apart
                    const __nv_bfloat16* src = (which == 0 ? p.Q : p.dY) + qoff + (rem / CH) * qstep;
                    const uint32_t dst = smem_u32(sStage + (it & 1) * L::STAGE_BYTES + which * (QBN * D * 2)) + rem * 16;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                                 "l"(reinterpret_cast<const uint4*>(src) + rem % CH)
                                 : "memory");
                }
            }
            if (next_tile > 0) {
                const int key0 = q0 + next_tile * QBN;
                for (int x = hslot; x < 4 * QBN * CH; x += PIPE_H_THREADS) {
                    const int plane = x / (QBN * CH), rem = x % (QBN * CH);
                    const __nv_bfloat16* base = plane == 0 ? gKa : plane == 1 ? gVa : plane == 2 ? gKb : gVb;
                    const uint32_t dst = smem_u32(sNext + (next_tile & 1) * L::NEXT_BYTES + plane * (QBN * D * 2)) + rem * 16;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                                 "l"(reinterpret_cast<const uint4*>(base + static_cast<size_t>(key0 + rem / CH) * kstep) + rem % CH)
                                 : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        h_stage(0, qoff_at(q0, 0), -1);
        fence_async_smem();
        cta_start_sync();
        constexpr int HB = 8;
        int n = 0, it = 0, n_tile_start = 0, ring_phase = 0;
        bool ok = true;
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int i0 = q0 + t * QBN;
            const bool prev_work = n > n_tile_start;      // the previous tile issued MMAs: Ring_free completes for it
            n_tile_start = n;
            const bool work = tile_has_work(i0);
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                asm volatile("cp.async.wait_all;" ::: "memory");
                warp_arrive(&bars[KB_H_SYNC], lane);
                ok = pipe_wait(&bars[KB_H_SYNC], it & 1, sFail);
                if (!ok) break;
                const bool boundary = hh == 0 && t > 0;
                if (boundary) {
                    const int knew = ring_key_w<W>(i0 + hg, hjs);
                    if (knew != kcur) {
                        kcur = knew;
                        const uint4* ka4 = reinterpret_cast<const uint4*>(next_row(0, knew));
                        const uint4* va4 = reinterpret_cast<const uint4*>(next_row(1, knew));
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const uint4 a = ka4[c], v = va4[c];
                            rKa[4 * c] = a.x; rKa[4 * c + 1] = a.y; rKa[4 * c + 2] = a.z; rKa[4 * c + 3] = a.w;
                            rVa[4 * c] = v.x; rVa[4 * c + 1] = v.y; rVa[4 * c + 2] = v.z; rVa[4 * c + 3] = v.w;
                        }
                    }
                }
                // The keys of tile t+1 go to the buffer tile t-1 used, which the other H warps may still be reading
                // at this tile's first head: they are requested at its second head (behind another H_sync).
                if (it + 1 < n_iter)
                    h_stage(it + 1, hh + 1 == G ? qoff_at(i0 + QBN, 0) : qoff_at(i0, hh + 1),
                            (hh == 1 && t + 1 < n_tiles) ? t + 1 : -1);
                const int qb = n & 1, gb = n & 1;
                uint8_t* dQp = sQp + qb * L::TILE;
                uint8_t* dG = sG + gb * L::TILE;
                const uint8_t* stage = sStage + (it & 1) * L::STAGE_BYTES;
                const uint4* q4 = reinterpret_cast<const uint4*>(stage + hg * (D * 2));
                const uint4* y4 = reinterpret_cast<const uint4*>(stage + QBN * D * 2 + hg * (D * 2));
                if (work) {
                    // Qp[n&1] was last read by the dKb MMAs of head n-2
                    if (n >= 2) ok = pipe_wait(&bars[KB_D_DONE0 + qb], ((n >> 1) - 1) & 1, sFail);
                    if (!ok) break;
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
                        }
                    }
                }
                if (boundary) {
                    // The own-side ring rows change key only after every MMA that reads them is done with the
                    // previous tile (the score-shaped products; Ring_free is committed behind the last of them).
                    if (prev_work) {
                        ok = pipe_wait(&bars[KB_RING_FREE], ring_phase & 1, sFail);
                        ++ring_phase;
                        if (!ok) break;
                    }
#pragma unroll
                    for (int x = hslot; x < 2 * QBN * CH; x += PIPE_H_THREADS) {
                        const int pl = x / (QBN * CH), rem = x % (QBN * CH), kr = rem / CH, c = rem % CH;
                        const int key = i0 + kr;
                        uint8_t* tile = pl == 0 ? sKb : sVb;
                        *reinterpret_cast<uint4*>(tile + sw128_offset<RING>(key & (RING - 1), c)) =
                            *reinterpret_cast<const uint4*>(next_row(2 + pl, key) + c * 16);
                    }
                }
                if (work || boundary) fence_async_smem();
                if (work) {
                    warp_arrive(&bars[KB_QP_FULL0 + qb], lane);
                    // Gt[n&1] was last read by the dVb MMAs of head n-2
                    if (n >= 2) ok = pipe_wait(&bars[KB_V_DONE0 + gb], ((n >> 1) - 1) & 1, sFail);
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
                    warp_arrive(&bars[KB_GT_FULL0 + gb], lane);
                    ++n;
                }
            }
        }
    } else if (warp >= 12) {
        reg_dec<M_REGS>();
        cta_start_sync();
        // Accumulator flushes: warp 12 + q reaches the tensor-memory lanes of quarter q.  The QBN lanes whose key
        // leaves at a tile boundary lie in one quarter (QBN divides 32 and tiles start on multiples of QBN).
        const int fslot = (warp & 3) * 32 + lane;
        const uint32_t tlf = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        auto acc_flush = [&](int lane_lo, int count, int i_ref, bool rezero) {
            flush_acc_range<D>(tlf, lane, lane_lo, count, ring_key(i_ref, fslot), gPartK, gPartV, p.scale, rezero);
        };
        const int n_bound = n_tiles - 1;
        if (!is_mma) {
            // ============================================================== flush warps (quarters 1-3)
            bool okf = true;
#pragma unroll 1
            for (int fb = 0; fb < n_bound && okf; ++fb) {
                const int i0 = q0 + (fb + 1) * QBN, s = i0 & (RING - 1);
                okf = pipe_wait(&bars[KB_ACC_DONE], fb & 1, sFail);     // every MMA of the tiles before this one is complete
                if (okf && (warp & 3) == (s >> 5)) {
                    tc_fence_after();
                    acc_flush(s & 31, QBN, i0 - 1, true);
                    warp_arrive(&bars[KB_FLUSH_DONE], lane);
                }
            }
            if (okf) okf = pipe_wait(&bars[KB_ACC_DONE], n_bound & 1, sFail);
            if (okf) {
                tc_fence_after();
                acc_flush(0, -1, q1 - 1, false);          // drain: every slot still holds a key of (q1 - 129, q1 - 1]
            }
        }
        if (is_mma) {
        // ================================================================== MMA warp
        const uint32_t issuer = elect_one();
        const uint32_t idesc_s = make_idesc_bf16(RING, RING, 0, 0);
        const uint32_t idesc_acc = make_idesc_bf16(RING, D, 0, 1);
        const uint64_t dKb = make_smem_desc(smem_u32(sKb), 16, 1024, SWIZZLE_128B);           // A, K-major
        const uint64_t dVb = make_smem_desc(smem_u32(sVb), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpK = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);          // B, K-major
        const uint64_t dGK = make_smem_desc(smem_u32(sG), 16, 1024, SWIZZLE_128B);
        const uint64_t dQpM = make_smem_desc(smem_u32(sQp), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major
        const uint64_t dGM = make_smem_desc(smem_u32(sG), RING * 128, 1024, SWIZZLE_128B);
        const uint32_t tAK = tmem_base + C_AK, tAV = tmem_base + C_AV;
        int n = 0, n_tile_start = 0, flushes_seen = 0;
        bool ok = true, flush_pending = false, dk_pending = false;
        auto a_col = [](int kk) -> uint32_t { return 64u * (kk >> 2) + 8u * (kk & 3); };
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
        int acc_commits = 0, self_i0 = 0;
        bool acc_commit_pending = false, self_pending = false;
        auto commit_acc = [&]() {
            umma_commit_pred(&bars[KB_ACC_DONE], issuer);
            ++acc_commits;
            acc_commit_pending = false;
        };
        auto issue_dk = [&](int m) {
            bool r = pipe_wait(&bars[KB_G_FULL], m & 1, sFail);
            if (r) {
                tc_fence_after();
                const uint32_t tA = tmem_base + C_R0 + (m & 1) * 128 + 32;
                const uint32_t qoff = (m & 1) * (L::TILE / 16);
                run_ts(tAK, tA, dQpM + qoff, 1);
                umma_commit_pred(&bars[KB_D_DONE0 + (m & 1)], issuer);
                if (acc_commit_pending) commit_acc();
            }
            return r;
        };
        auto settle_flush = [&]() {
            bool r = true;
            if (flush_pending) {
                r = pipe_wait(&bars[KB_FLUSH_DONE], flushes_seen & 1, sFail);
                ++flushes_seen;
                flush_pending = false;
                if (r) tc_fence_after();
            }
            if (r && self_pending) {
                r = pipe_wait(&bars[KB_ACC_DONE], (acc_commits - 1) & 1, sFail);
                self_pending = false;
                if (r) {
                    tc_fence_after();
                    acc_flush(self_i0 & 31, QBN, self_i0 - 1, true);
                    __syncwarp();
                    tc_fence_after();
                }
            }
            return r;
        };
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int i0 = q0 + t * QBN;
            if (t > 0) {
                if (flush_pending || self_pending) {
                    if (dk_pending) { ok = issue_dk(n - 1); dk_pending = false; }
                    if (ok) ok = settle_flush();
                    if (!ok) break;
                }
                if (((i0 & (RING - 1)) >> 5) == 0) { self_pending = true; self_i0 = i0; }
                else flush_pending = true;
                if (dk_pending) acc_commit_pending = true;   // committed right behind the kept-back dKb MMAs
                else commit_acc();
            }
            const bool work = tile_has_work(i0);
            bool ring_committed = false;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                if (!work) {
                    if (dk_pending) { ok = issue_dk(n - 1); dk_pending = false; }
                    continue;
                }
                const uint32_t ph = n & 1;
                const int qb = n & 1, gb = n & 1;
                const uint32_t qoff = qb * (L::TILE / 16), goff = gb * (L::TILE / 16);
                const uint32_t tA = tmem_base + C_R0 + (n & 1) * 128;          // X^T, then P^T | gA^T
                const uint32_t tB = tmem_base + C_R0 + ((n & 1) ^ 1) * 128;    // dP^T
                ok = pipe_wait(&bars[KB_QP_FULL0 + qb], (n >> 1) & 1, sFail);
                if (ok && n > 0) ok = pipe_wait(&bars[KB_B_FREE], (n - 1) & 1, sFail);
                if (!ok) break;
                tc_fence_after();
                run_ss(tA, dKb, dQpK + qoff);                  // X^T = Kb Qp^T
                umma_commit_pred(&bars[KB_S_XT], issuer);
                if (dk_pending) {
                    ok = issue_dk(n - 1);
                    dk_pending = false;
                    if (!ok) break;
                }
                if (n > 0) ok = pipe_wait(&bars[KB_D_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail);
                if (ok) ok = pipe_wait(&bars[KB_GT_FULL0 + gb], (n >> 1) & 1, sFail);
                if (!ok) break;
                tc_fence_after();
                run_ss(tB, dVb, dGK + goff);                   // dP^T = Vb Gt^T
                umma_commit_pred(&bars[KB_S_DP], issuer);
                if (hh == G - 1) {
                    umma_commit_pred(&bars[KB_RING_FREE], issuer);
                    ring_committed = true;
                }
                ok = pipe_wait(&bars[KB_P_FULL], ph, sFail);
                if (ok && (flush_pending || self_pending)) ok = settle_flush();   // the lanes zeroed at the tile boundary
                if (!ok) break;
                tc_fence_after();
                run_ts(tAV, tA, dGM + goff, 1);                // dVb += P^T Gt
                umma_commit_pred(&bars[KB_V_DONE0 + gb], issuer);
                dk_pending = true;
                ++n;
            }
            if (n > n_tile_start && ok && !ring_committed) umma_commit_pred(&bars[KB_RING_FREE], issuer);
            n_tile_start = n;
        }
        if (ok && dk_pending) ok = issue_dk(n - 1);
        if (ok) ok = settle_flush();
        if (ok) {
            commit_acc();
            ok = pipe_wait(&bars[KB_ACC_DONE], (acc_commits - 1) & 1, sFail);
            if (ok) {
                tc_fence_after();
                acc_flush(0, -1, q1 - 1, false);
            }
        }
        __syncwarp();
        }
    } else {
        // ================================================================== E warps
        reg_dec<E_REGS>();
        cta_start_sync();
        const int slot = tid & (RING - 1);               // tensor-memory lane = own-side ring slot
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
        // Per-head constants of the NG queries whose columns this thread's half holds: lane q < NG fetches those
        // of query i0 + ch * NG + q one head ahead; the values are broadcast by shuffles where they are used.
        float pre_m = 0.f, pre_l = 0.f, pre_d = 0.f;
        auto prefetch = [&](int i0, int hh) {
            if (lane < NG) {
                const size_t row = row_at(i0 + ch * NG + lane, hh);
                pre_m = __ldg(p.m + row); pre_l = __ldg(p.l + row); pre_d = __ldg(p.delta + row);
            }
        };
        prefetch(q0, 0);
        int n = 0;
        bool ok = true;
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int i0 = q0 + t * QBN, i_last = i0 + QBN - 1;
            // Visibility.  For each of this half's NG queries: the four words over the 128 own-side slots (the
            // query's visible keys), from which follow this lane's own-key bit, the query's visible-key count and,
            // because both key axes see the same keys, the bits of its W columns.
            uint32_t kvis = 0, single = 0, live_vis = 0;      // bit q: per query of this half
            uint32_t colw[2] = {0, 0};                        // bit c of word cc: column cc*32 + c holds a visible key
            bool any_work = false;
#pragma unroll
            for (int q = 0; q < NG; ++q) {
                const int i = i0 + ch * NG + q;
                uint32_t vw[4];
                column_visibility(mask_b.row(i), i, i_last, p.window, lane, vw);
                const int nv = __popc(vw[0]) + __popc(vw[1]) + __popc(vw[2]) + __popc(vw[3]);
                if (nv > 0) live_vis |= 1u << q;
                if (nv == 1) single |= 1u << q;
                if ((vw[slot >> 5] >> (slot & 31)) & 1u) kvis |= 1u << q;
                // columns of this query inside the half: W consecutive columns starting at q * W
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int c = cc * 32 + lane;             // column within the half this lane evaluates
                    bool v = false;
                    if (c / W == q) {
                        const int kj = ring_key_w<W>(i, c & (W - 1));
                        v = kj >= 0 && ((vw[(kj & (RING - 1)) >> 5] >> (kj & 31)) & 1u);
                    }
                    colw[cc] |= __ballot_sync(0xFFFFFFFFu, v);
                }
            }
            if (mask_b.any()) {
                any_work = tile_has_work(i0);
            } else {
                any_work = true;
            }
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                // constants of this head, broadcast from the lanes that fetched them
                float lse2[NG], dlt[NG];
                uint32_t live = 0;
#pragma unroll
                for (int q = 0; q < NG; ++q) {
                    const float m_q = __shfl_sync(0xFFFFFFFFu, pre_m, q), l_q = __shfl_sync(0xFFFFFFFFu, pre_l, q);
                    dlt[q] = __shfl_sync(0xFFFFFFFFu, pre_d, q);
                    const bool lv = ((live_vis >> q) & 1u) && l_q > 0.f;
                    lse2[q] = lv ? m_q * LOG2E + __log2f(l_q) : 0.f;
                    if (lv) live |= 1u << q;
                }
                if (hh + 1 < G) prefetch(i0, hh + 1);
                else if (t + 1 < n_tiles) prefetch(i0 + QBN, 0);
                if (!any_work) continue;
                // this thread's cell mask: column holds a visible key, the column's query is live and sees this lane's key
                uint32_t cw[2];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t qmask = 0;
#pragma unroll
                    for (int q = 0; q < NG; ++q) {
                        // columns of query q inside word cc
                        const int lo = q * W - cc * 32, hi = lo + W;
                        if (hi > 0 && lo < 32 && ((kvis & live) >> q) & 1u) {
                            const int a = lo < 0 ? 0 : lo, e = hi > 32 ? 32 : hi;
                            qmask |= (e - a == 32) ? 0xFFFFFFFFu : (((1u << (e - a)) - 1u) << a);
                        }
                    }
                    cw[cc] = colw[cc] & qmask;
                }
                const uint32_t ph = n & 1;
                const uint32_t tA = tl + C_R0 + (n & 1) * 128 + ch * 64;          // this thread's 64 score columns
                const uint32_t tB = tl + C_R0 + ((n & 1) ^ 1) * 128;
                // ---- phase 1: P^T = exp2(X^T c2 - lse) for this thread's 64 columns, BF16 into the first 32
                ok = pipe_wait(&bars[KB_S_XT], ph, sFail);
                if (!ok) break;
                tc_fence_after();
                const uint64_t c2p = pair_f32(c2, c2);
                const bool warp0 = __ballot_sync(0xFFFFFFFFu, cw[0] != 0) != 0, warp1 = __ballot_sync(0xFFFFFFFFu, cw[1] != 0) != 0;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t pk[16];
                    if (!(cc ? warp1 : warp0)) {              // no lane of this warp has a live cell in these 32 columns
#pragma unroll
                        for (int t4 = 0; t4 < 16; ++t4) pk[t4] = 0u;
                    } else {
                        uint32_t x[32];
                        tmem_ld32(tA + cc * 32, x);
                        tmem_wait_ld();
                        const uint32_t w = cw[cc];
#pragma unroll
                        for (int t4 = 0; t4 < 32; t4 += 2) {
                            const float ls = lse2[(cc * 32 + t4) / W];
                            float a0, a1;                     // packed FP32: two columns an instruction
                            unpair_f32(fma_f32x2(pair_b32(x[t4], x[t4 + 1]), c2p, pair_f32(-ls, -ls)), a0, a1);
                            float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                            if (!((w >> t4) & 1u)) p0 = 0.f;
                            if (!((w >> (t4 + 1)) & 1u)) p1 = 0.f;
                            pk[t4 >> 1] = pack_bf16x2(p0, p1);
                        }
                    }
                    tmem_st16(tA + cc * 16, pk);
                }
                tmem_wait_st();
                tc_fence_before();
                warp_arrive(&bars[KB_P_FULL], lane);
                // ---- phase 2: gA^T = P^T o (dP^T - delta), BF16 into the last 32 of this thread's columns
                ok = pipe_wait(&bars[KB_S_DP], ph, sFail);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t pk[16];
                    const bool act = cc ? warp1 : warp0;
                    if (act) {
                        uint32_t dp[32];
                        tmem_ld32(tB + ch * 64 + cc * 32, dp);
                        tmem_ld16(tA + cc * 16, pk);
                        tmem_wait_ld();
#pragma unroll
                        for (int t4 = 0; t4 < 32; t4 += 2) {
                            const int q = (cc * 32 + t4) / W;
                            float d0, d1;
                            unpair_f32(add_f32x2(pair_b32(dp[t4], dp[t4 + 1]), pair_f32(-dlt[q], -dlt[q])), d0, d1);
                            const uint32_t d2 = pack_bf16x2(d0, d1);
                            pk[t4 >> 1] = ((single >> q) & 1u) ? 0u : mul_bf16x2(pk[t4 >> 1], d2);
                        }
                    } else {
#pragma unroll
                        for (int t4 = 0; t4 < 16; ++t4) pk[t4] = 0u;
                    }
                    if (cc == 1) {
                        // dP^T is in registers (or not needed): the next head's scores may land on these columns
                        tc_fence_before();
                        warp_arrive(&bars[KB_B_FREE], lane);
                    }
                    tmem_st16(tA + 32 + cc * 16, pk);
                }
                tmem_wait_st();
                tc_fence_before();
                warp_arrive(&bars[KB_G_FULL], lane);
                ++n;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*sFail && tid == 0) atomicExch(p.status, 300 + *sFail);
    if (is_mma) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace sgpack
