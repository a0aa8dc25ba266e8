// Self-test of the tcgen05 building blocks the triplet kernels rely on: one CTA
// multiplies two 128x128 BF16 matrices through each operand arrangement the
// kernels use (K-major and MN-major shared-memory operands in the 128-byte
// swizzle, and an A operand held in tensor memory) and returns the FP32
// accumulator, so the descriptor encodings can be checked against a plain
// matrix product on the host.  The encodings are the ones the kernels use and
// are fixed here; nothing about a descriptor comes from the caller.
#include "sm100_ptx.cuh"
#include "att3_abi_internal.h"

using namespace sm100;

namespace {

constexpr int T = 128;            // tile edge: M = N = K = 128
constexpr int TILE_BYTES = T * T * 2;

// Leading / stride byte offsets of the two operand arrangements (128-byte swizzle, 128-row tiles):
// K-major: 8-row groups 1024 bytes apart, the leading offset is unused by the hardware (16);
// MN-major: the next 64-element block along M/N is a whole [128][64] slab away (16384), 8 K-rows 1024.
constexpr uint32_t LBO_K = 16, SBO_K = 1024, LBO_MN = T * 128, SBO_MN = 1024;

struct SelftestParams {
    const __nv_bfloat16* A;       // [128][128] row-major
    const __nv_bfloat16* B;       // [128][128] row-major
    float* D;                     // [128][128] row-major
    int mode;
    int* status;
};

// mode 0: D[m][n] = sum_k A[m][k] * B[n][k]   (A, B both K-major in smem)
// mode 1: D[m][n] = sum_k A[m][k] * B[k][n]   (A K-major, B MN-major)
// mode 2: D[m][n] = sum_k A[k][m] * B[k][n]   (A, B both MN-major)
// mode 3: D[m][n] = sum_k A[m][k] * B[k][n]   (A in tensor memory, B MN-major)
// mode 4: D[m][n] = sum_k A[m][k] * B[n][k]   (A in tensor memory, B K-major)
// mode | 8: the same product as an N = 64 instruction (first 64 output columns).
__global__ void __launch_bounds__(128, 1) umma_selftest_kernel(SelftestParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment keeps the swizzle phase equal to (row & 7).
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + TILE_BYTES;
    __shared__ uint64_t mma_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_ok;

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
    {   // one row of each matrix per thread, 16-byte chunks into the swizzled tile
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

    const int nwidth = (p.mode & 8) ? 64 : T;
    const int mode = p.mode & 7;
    const bool a_in_tmem = (mode == 3 || mode == 4);
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

    if (tid == 0) {
        tc_fence_after();
        const int a_mn = (mode == 2) ? 1 : 0;
        const int b_mn = (mode == 1 || mode == 2 || mode == 3) ? 1 : 0;
        const uint32_t idesc = make_idesc_bf16(T, nwidth, a_mn, b_mn);
        const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB);
#pragma unroll 1
        for (int kk = 0; kk < T / 16; ++kk) {
            // K-major: 16 K-elements = 32 bytes inside the 128-byte line, next d_block every 4 steps.
            // MN-major: 16 K-rows = two 8-row groups = 2048 bytes.
            const uint32_t a_off = a_mn ? kk * 2048 : (kk >> 2) * (T * 128) + (kk & 3) * 32;
            const uint32_t b_off = b_mn ? kk * 2048 : (kk >> 2) * (T * 128) + (kk & 3) * 32;
            const uint64_t bdesc = make_smem_desc(b_base + b_off, b_mn ? LBO_MN : LBO_K, b_mn ? SBO_MN : SBO_K, SWIZZLE_128B);
            if (a_in_tmem) {
                umma_ts(tmem_d, tmem_a + kk * 8, bdesc, idesc, kk > 0);
            } else {
                const uint64_t adesc = make_smem_desc(a_base + a_off, a_mn ? LBO_MN : LBO_K, a_mn ? SBO_MN : SBO_K, SWIZZLE_128B);
                umma_ss(tmem_d, adesc, bdesc, idesc, kk > 0);
            }
        }
        umma_commit(&mma_bar);
        s_ok = mbar_wait(&mma_bar, 0) ? 1 : 0;      // bounded: a logic error ends with a status, not a hang
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    tc_fence_after();
    if (!ok) {
        if ((tid & 31) == 0) atomicExch(p.status, 1);
    } else {
        uint32_t r[32];
#pragma unroll 1
        for (int c = 0; c < nwidth / 32; ++c) {
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

extern "C" int att3_umma_selftest(const void* A, const void* B, float* D, int mode, int* status_dev, void* stream) {
    if (!A || !B || !D || !status_dev) return att3::set_error(ATT3_ERR_INVALID, "umma_selftest: null pointer");
    if (mode < 0 || (mode & 7) > 4 || mode > 15)
        return att3::set_error(ATT3_ERR_INVALID, "umma_selftest: mode must be 0..4 (+8: N = 64)");
    if (!att3::require_sm100("umma_selftest")) return ATT3_ERR_UNSUPPORTED;
    SelftestParams p;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.B = static_cast<const __nv_bfloat16*>(B);
    p.D = D;
    p.mode = mode;
    p.status = status_dev;
    const int smem = 2 * TILE_BYTES + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return att3::set_cuda_error(e, "umma_selftest: smem opt-in");
    umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "umma_selftest: launch");
    return ATT3_OK;
}
