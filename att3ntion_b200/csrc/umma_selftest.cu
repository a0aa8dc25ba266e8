// Self-test of the tcgen05 building blocks the triplet kernels rely on: one CTA
// multiplies two 128x128 BF16 matrices through each operand arrangement the
// kernels use (K-major and MN-major shared-memory operands in the 128-byte
// swizzle, and an A operand held in tensor memory) and returns the FP32
// accumulator, so the descriptor encodings can be checked against a plain
// matrix product on the host.
#include "sm100_ptx.cuh"
#include "att3_abi_internal.h"

using namespace sm100;

namespace {

constexpr int T = 128;            // tile edge: M = N = K = 128
constexpr int TILE_BYTES = T * T * 2;

struct SelftestParams {
    const __nv_bfloat16* A;       // [128][128] row-major
    const __nv_bfloat16* B;       // [128][128] row-major
    float* D;                     // [128][128] row-major
    int mode;
    uint32_t lbo_a, sbo_a, lbo_b, sbo_b;
    int reps;
    int tight;                    // mode | 16: converged-warp issue with precomputed descriptors
    int* status;
};

// mode 0: D[m][n] = sum_k A[m][k] * B[n][k]   (A, B both K-major in smem)
// mode 1: D[m][n] = sum_k A[m][k] * B[k][n]   (A K-major, B MN-major)
// mode 2: D[m][n] = sum_k A[k][m] * B[k][n]   (A, B both MN-major)
// mode 3: D[m][n] = sum_k A[m][k] * B[k][n]   (A in tensor memory, B MN-major)
// mode 4: D[m][n] = sum_k A[m][k] * B[n][k]   (A in tensor memory, B K-major)
__global__ void __launch_bounds__(128, 1) umma_selftest_kernel(SelftestParams p) {
    long long t_issue = 0;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment keeps the swizzle phase equal to (row & 7).
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + TILE_BYTES;
    __shared__ uint64_t mma_bar;
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;

    if (warp == 0) {
        tmem_alloc(&tmem_base_slot, 256);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&mma_bar, 1);
        fence_mbar_init();
    }
    // One row of each matrix per thread, 16-byte chunks into the swizzled tile.
    {
        const uint4* ga = reinterpret_cast<const uint4*>(p.A + tid * T);
        const uint4* gb = reinterpret_cast<const uint4*>(p.B + tid * T);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            *reinterpret_cast<uint4*>(sA + sw128_offset<T>(tid, c)) = ga[c];
            *reinterpret_cast<uint4*>(sB + sw128_offset<T>(tid, c)) = gb[c];
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_d = tmem_base;            // columns [0,128): accumulator
    const uint32_t tmem_a = tmem_base + 128;      // columns [128,192): packed BF16 A operand
    const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;

    const int nwidth = (p.mode & 8) ? 64 : T;       // mode | 8: the same product restricted to N = 64 columns
    p.tight = (p.mode >> 4) & 1;                      // converged warp, one elected lane, precomputed descriptors
    p.mode &= 7;
    const bool a_in_tmem = (p.mode == 3 || p.mode == 4);
    if (a_in_tmem) {
        // Thread m holds row m of A: 128 BF16 = 64 packed words = columns [0,64) of the A region.
        const uint32_t* ga = reinterpret_cast<const uint32_t*>(p.A + tid * T);
        uint32_t r[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = ga[half * 32 + i];
            tmem_st32(tmem_a + lane_field + half * 32, r);
        }
        tmem_wait_st();
        tc_fence_before();
    }
    __syncthreads();

    if (p.tight && warp == 0) {
        // Rate probe: whole warp converged, descriptor bases precomputed, k-steps unrolled.
        tc_fence_after();
        const int b_mn = (p.mode == 1 || p.mode == 3) ? 1 : 0;
        const uint32_t idesc = make_idesc_bf16(T, nwidth, 0, b_mn);
        const uint64_t da = make_smem_desc(smem_u32(sA), p.lbo_a, p.sbo_a, SWIZZLE_128B);
        const uint64_t db = make_smem_desc(smem_u32(sB), p.lbo_b, p.sbo_b, SWIZZLE_128B);
        const uint32_t issuer = elect_one();
        const long long t0 = clock64();
        for (int rep = 0; rep < p.reps; ++rep) {
#pragma unroll
            for (int kk = 0; kk < T / 16; ++kk) {
                const uint32_t koff = ((kk >> 2) * (T * 128) + (kk & 3) * 32) / 16;
                const uint32_t moff = kk * 2048 / 16;
                const uint32_t acc = (rep > 0 || kk > 0) ? 1u : 0u;
                if (a_in_tmem) umma_ts_pred(tmem_d, tmem_a + kk * 8, db + (b_mn ? moff : koff), idesc, acc, issuer);
                else umma_ss_pred(tmem_d, da + koff, db + (b_mn ? moff : koff), idesc, acc, issuer);
            }
        }
        const long long t1 = clock64();
        umma_commit_pred(&mma_bar, issuer);
        if (tid == 0) { p.status[2] = static_cast<int>(t1 - t0); t_issue = t0; }
    } else if (!p.tight && tid == 0) {
        tc_fence_after();
        const int a_mn = (p.mode == 2) ? 1 : 0;
        const int b_mn = (p.mode == 1 || p.mode == 2 || p.mode == 3) ? 1 : 0;
        const uint32_t idesc = make_idesc_bf16(T, nwidth, a_mn, b_mn);
        t_issue = clock64();
        const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB);
        for (int rep = 0; rep < p.reps; ++rep) {
#pragma unroll 1
            for (int kk = 0; kk < T / 16; ++kk) {
                // K-major: 16 K-elements = 32 bytes inside the 128-byte line, next d_block every 4 steps.
                // MN-major: 16 K-rows = two 8-row groups = 2048 bytes.
                const uint32_t a_off = a_mn ? kk * 2048 : (kk >> 2) * (T * 128) + (kk & 3) * 32;
                const uint32_t b_off = b_mn ? kk * 2048 : (kk >> 2) * (T * 128) + (kk & 3) * 32;
                const uint64_t bdesc = make_smem_desc(b_base + b_off, p.lbo_b, p.sbo_b, SWIZZLE_128B);
                const uint32_t acc = (rep > 0 || kk > 0) ? 1u : 0u;
                if (a_in_tmem) {
                    umma_ts(tmem_d, tmem_a + kk * 8, bdesc, idesc, acc);
                } else {
                    const uint64_t adesc = make_smem_desc(a_base + a_off, p.lbo_a, p.sbo_a, SWIZZLE_128B);
                    umma_ss(tmem_d, adesc, bdesc, idesc, acc);
                }
            }
        }
        const long long t_issued = clock64();
        umma_commit(&mma_bar);
        p.status[2] = static_cast<int>(t_issued - t_issue);              // cycles spent issuing
    }
    // Only the issuing thread polls; the others park at the CTA barrier so that nothing
    // competes with the operand traffic while the rate is measured.
    __shared__ int s_ok;
    if (tid == 0) {
        s_ok = mbar_wait(&mma_bar, 0) ? 1 : 0;
        p.status[1] = static_cast<int>(clock64() - t_issue);             // cycles from first issue to completion
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    tc_fence_after();
    if (!ok) {
        if ((tid & 31) == 0) atomicExch(p.status, 1);
    } else {
        uint32_t r[32];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            tmem_ld32(tmem_d + lane_field + c * 32, r);
            tmem_wait_ld();
            float4* dst = reinterpret_cast<float4*>(p.D + tid * T + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                     __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace

extern "C" int att3_umma_selftest(const void* A, const void* B, float* D, int mode, int lbo_a, int sbo_a,
                                  int lbo_b, int sbo_b, int reps, int* status_dev, void* stream) {
    if (!A || !B || !D || !status_dev) return att3::set_error(ATT3_ERR_INVALID, "umma_selftest: null pointer");
    if ((mode & 7) > 4 || mode < 0 || mode > 31 || ((mode & 16) && (mode & 7) == 2) || reps < 1 || reps > 64)
        return att3::set_error(ATT3_ERR_INVALID, "umma_selftest: mode must be 0..4 (+8: N = 64, +16: converged-warp issue) and reps 1..64");
    SelftestParams p;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.B = static_cast<const __nv_bfloat16*>(B);
    p.D = D;
    p.mode = mode;
    p.lbo_a = lbo_a; p.sbo_a = sbo_a; p.lbo_b = lbo_b; p.sbo_b = sbo_b;
    p.reps = reps;
    p.tight = 0;
    p.status = status_dev;
    const int smem = 2 * TILE_BYTES + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return att3::set_cuda_error(e, "umma_selftest: smem opt-in");
    umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "umma_selftest: launch");
    return ATT3_OK;
}

// ---------------------------------------------------------------------------
// Diagnostic (not in the public header): cycles per tcgen05.mma as seen by the issuing thread,
// for several ways of writing the issue loop.  With N = 16 an MMA occupies the tensor pipe for a
// few cycles only, so the figure is the issue cost itself; with N = 128 it is max(issue, 64).
//   style 0  lane-0 branch, every operand a compile-time function of the shared-memory base
//   style 1  lane-0 branch, descriptors and tensor-memory addresses offset by per-thread values
//            (what a buffer index derived from a data-dependent loop counter looks like)
//   style 2  as 1, the values passed through a shuffle from lane 0 (marks them warp-uniform)
//   style 3  whole warp converged, one lane elected once, MMAs predicated on it; operands as in 2
//   style 4  as 3 with the per-thread operands of style 1
// ---------------------------------------------------------------------------
namespace {

template <int STYLE, bool TS, int NW>
__global__ void __launch_bounds__(128, 1) umma_rate_kernel(int* status, int reps) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + TILE_BYTES;
    __shared__ uint64_t mma_bar;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp == 0) {
        tmem_alloc(&tmem_base_slot, 256);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&mma_bar, 1);
        fence_mbar_init();
    }
    for (int c = 0; c < 16; ++c) {
        *reinterpret_cast<uint4*>(sA + tid * 256 + c * 16) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sB + tid * 256 + c * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) {
        uint32_t tmem_base = tmem_base_slot;
        uint32_t roff = static_cast<uint32_t>(status[3]);      // zero, but only known at run time, per thread
        if (STYLE == 0) roff = 0;
        if (STYLE == 2 || STYLE == 3) {
            roff = __shfl_sync(0xFFFFFFFFu, roff, 0);
            tmem_base = __shfl_sync(0xFFFFFFFFu, tmem_base, 0);
        }
        const uint32_t idesc = make_idesc_bf16(T, NW, 0, 0);
        const uint64_t da = make_smem_desc(smem_u32(sA), 16, 1024, SWIZZLE_128B) + roff;
        const uint64_t db = make_smem_desc(smem_u32(sB), 16, 1024, SWIZZLE_128B) + roff;
        const uint32_t tD = tmem_base + roff, tA = tmem_base + 128 + roff;
        long long t0 = 0, t1 = 0;
        if (STYLE <= 2) {
            if (lane == 0) {
                t0 = clock64();
#pragma unroll 1
                for (int rep = 0; rep < reps; ++rep) {
#pragma unroll
                    for (int kk = 0; kk < T / 16; ++kk) {
                        const uint32_t koff = ((kk >> 2) * (T * 128) + (kk & 3) * 32) / 16;
                        if (TS) umma_ts(tD, tA + kk * 8, db + koff, idesc, kk > 0);
                        else umma_ss(tD, da + koff, db + koff, idesc, kk > 0);
                    }
                }
                t1 = clock64();
                umma_commit(&mma_bar);
            }
            __syncwarp();
        } else {
            const uint32_t elected = elect_one();
            t0 = clock64();
#pragma unroll 1
            for (int rep = 0; rep < reps; ++rep) {
#pragma unroll
                for (int kk = 0; kk < T / 16; ++kk) {
                    const uint32_t koff = ((kk >> 2) * (T * 128) + (kk & 3) * 32) / 16;
                    if (TS) umma_ts_pred(tD, tA + kk * 8, db + koff, idesc, kk > 0, elected);
                    else umma_ss_pred(tD, da + koff, db + koff, idesc, kk > 0, elected);
                }
            }
            t1 = clock64();
            if (elected) umma_commit(&mma_bar);
            __syncwarp();
        }
        if (lane == 0) {
            status[2] = static_cast<int>(t1 - t0);
            status[0] = mbar_wait(&mma_bar, 0) ? 0 : 1;
            status[1] = static_cast<int>(clock64() - t0);
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base_slot, 256);
}

template <int STYLE, bool TS>
int launch_rate(int nw, int* status, int reps, cudaStream_t st) {
    const int smem = 2 * TILE_BYTES + 1024;
    auto go = [&](auto kern) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "umma_rate: smem opt-in");
        kern<<<1, 128, smem, st>>>(status, reps);
        e = cudaGetLastError();
        return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "umma_rate: launch");
    };
    return nw == 16 ? go(umma_rate_kernel<STYLE, TS, 16>) : go(umma_rate_kernel<STYLE, TS, 128>);
}

}  // namespace

extern "C" int att3_debug_mma_rate(int style, int ts, int nwidth, int reps, int* status_dev, void* stream) {
    if (!att3::require_sm100("umma_rate")) return ATT3_ERR_UNSUPPORTED;
    if (style < 0 || style > 4 || (nwidth != 16 && nwidth != 128) || reps < 1 || reps > 4096 || !status_dev)
        return att3::set_error(ATT3_ERR_INVALID, "umma_rate: style 0..4, nwidth 16|128, reps 1..4096");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (style * 2 + (ts ? 1 : 0)) {
        case 0: return launch_rate<0, false>(nwidth, status_dev, reps, st);
        case 1: return launch_rate<0, true>(nwidth, status_dev, reps, st);
        case 2: return launch_rate<1, false>(nwidth, status_dev, reps, st);
        case 3: return launch_rate<1, true>(nwidth, status_dev, reps, st);
        case 4: return launch_rate<2, false>(nwidth, status_dev, reps, st);
        case 5: return launch_rate<2, true>(nwidth, status_dev, reps, st);
        case 6: return launch_rate<3, false>(nwidth, status_dev, reps, st);
        case 7: return launch_rate<3, true>(nwidth, status_dev, reps, st);
        case 8: return launch_rate<4, false>(nwidth, status_dev, reps, st);
        default: return launch_rate<4, true>(nwidth, status_dev, reps, st);
    }
}
