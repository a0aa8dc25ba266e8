// C-ABI entry points of the single query gather (independent and shared KV
// heads): argument validation, query-block partitioning and kernel launches.
#include <algorithm>
#include <cmath>

#include "att3_abi_internal.h"
#include "sg_ring_fwd.cuh"

namespace {

// Sticky status word of this translation unit's kernels (bounded-wait failures).
__device__ int g_sg_status = 0;

int* status_ptr() {
    int* p = nullptr;
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sg_status);
    return p;
}

// Validation shared by forward and backward; mirrors single_gather_check and
// single_gather_shared_check of the reference (cuda/forward.cu:1609-1653).
int check_shapes(const char* who, int B, int Hq, int Hkv, int N, int D, int window, int q_begin) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: empty batch/head dimensions are unsupported", who);
    if (N <= 0 || N % 16 != 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: N must be a positive multiple of 16, got %d", who, N);
    if (D != 64 && D != 128) return att3::set_error(ATT3_ERR_INVALID, "%s: D must be 64 or 128, got %d", who, D);
    if (Hq % Hkv != 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: Hq=%d is not divisible by Hkv=%d", who, Hq, Hkv);
    if (window < 0 || window > sgring::RING)
        return att3::set_error(ATT3_ERR_INVALID, "%s: window must be in [0,128], got %d", who, window);
    if (q_begin < 0 || q_begin >= N)
        return att3::set_error(ATT3_ERR_INVALID, "%s: q_begin must be in [0,N), got %d", who, q_begin);
    return ATT3_OK;
}

// Query-block partition of the ring kernels: as many CTAs as the device holds
// at `ctas_per_sm` residency, never shorter than `min_len` queries per block.
int plan_blocks(int B, int Hkv, int N, int q_begin, int sm_count, int ctas_per_sm, int min_len, int* block_len) {
    const int nq = N - q_begin;
    const int slots = std::max(1, sm_count * ctas_per_sm);
    int nblk = std::max(1, slots / std::max(1, B * Hkv));
    int len = (nq + nblk - 1) / nblk;
    len = std::max(len, std::min(min_len, nq));
    nblk = (nq + len - 1) / len;
    *block_len = len;
    return nblk;
}

}  // namespace

extern "C" int att3_sg_query_blocks(int B, int Hq, int Hkv, int N, int q_begin, int sm_count, int* block_len) {
    (void)Hq;
    int len = 0;
    const int n = plan_blocks(B, Hkv, N, q_begin, sm_count, 2, 16, &len);
    if (block_len) *block_len = len;
    return n * B * Hkv;
}

extern "C" int att3_device_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_device_status: synchronize");
    int h = 0;
    e = cudaMemcpyFromSymbol(&h, g_sg_status, sizeof(int));
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_device_status: read");
    if (h != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_sg_status, &zero, sizeof(int));
        return att3::set_error(ATT3_ERR_TIMEOUT, "a bounded device-side wait ran out (status %d)", h);
    }
    return ATT3_OK;
}

template <int D>
static int launch_ring_fwd(const sgring::FwdParams& p, int nblk, cudaStream_t stream) {
    using L = sgring::FwdSmem<D>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(sgring::sg_ring_fwd_kernel<D>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_forward: shared-memory opt-in");
        configured_dev = dev;
    }
    dim3 grid(nblk, p.Hkv, p.B);
    sgring::sg_ring_fwd_kernel<D><<<grid, sgring::NTHREADS, L::ALLOC, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_forward: launch");
    att3::count_launch(0);
    return ATT3_OK;
}

extern "C" int att3_sg_forward(const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                               const uint8_t* mask, void* Y, float* m, float* l, int B, int Hq, int Hkv, int N,
                               int D, int window, int q_begin, void* stream) {
    if (int rc = check_shapes("att3_sg_forward", B, Hq, Hkv, N, D, window, q_begin)) return rc;
    if (!Q || !R || !S || !Vr || !Vs || !Y || !m || !l)
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_forward: null tensor pointer");
    if (!att3::require_sm100("att3_sg_forward")) return ATT3_ERR_UNSUPPORTED;
    if (window == 0)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_sg_forward: dense (window = 0) path not built");
    sgring::FwdParams p;
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.R = static_cast<const __nv_bfloat16*>(R);
    p.S = static_cast<const __nv_bfloat16*>(S);
    p.Vr = static_cast<const __nv_bfloat16*>(Vr);
    p.Vs = static_cast<const __nv_bfloat16*>(Vs);
    p.mask = mask;
    p.Y = static_cast<__nv_bfloat16*>(Y);
    p.m = m;
    p.l = l;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.window = window; p.q_begin = q_begin;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = status_ptr();
    const int nblk = plan_blocks(B, Hkv, N, q_begin, att3::sm_count(), 2, 16, &p.block_len);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return D == 64 ? launch_ring_fwd<64>(p, nblk, st) : launch_ring_fwd<128>(p, nblk, st);
}
