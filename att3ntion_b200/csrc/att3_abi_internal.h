// Error plumbing shared by the translation units behind the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/att3_b200.h"

namespace att3 {

// Records `msg` as the calling thread's last error and returns `code`.
int set_error(int code, const char* fmt, ...);
int set_cuda_error(cudaError_t e, const char* where);

// True when the current device can run the sm_100a kernels; otherwise records
// ATT3_ERR_UNSUPPORTED with the reason.
bool require_sm100(const char* who);

// Streaming multiprocessor count of the current device (cached per device).
int sm_count();

// Launch counters behind att3_launch_count().
void count_launch(int which, int n = 1);

// Kernel ids of att3_timing_read().
enum KernelId { K_SG_FWD = 0, K_SG_BWD = 1, K_SG_REDUCE = 2, K_DENSE_FWD = 3, K_DENSE_BWD = 4, K_HG_AUX = 5, K_COUNT = 6 };

// Brackets one kernel launch with CUDA events on its stream while timing is
// enabled (att3_timing_enable); a no-op otherwise.
class TimedLaunch {
public:
    TimedLaunch(int kernel_id, cudaStream_t stream);
    ~TimedLaunch();
private:
    int id_;
    cudaStream_t stream_;
    cudaEvent_t start_ = nullptr;
};

// Tensor map over a row-major BF16 matrix [rows, cols] whose TMA box is `box_rows` whole rows (cols <= 256):
// the descriptor behind the kernels' row staging.  Encoded through the driver entry point obtained from
// the runtime (no link-time dependency on the driver library).  Returns ATT3_OK or records the error.
int make_row_tensor_map(CUtensorMap* out, const void* base, size_t rows, int cols, const char* who, int box_rows = 1,
                        int pitch_cols = 0);
// The same over a [B,H,N,D] operand in either memory layout (0: [B,H,N,D] -> [B*H*N, D]; 1: [B,N,H,D] -> [B*N, H*D],
// the head being a column offset of the box): the (x, y) a kernel passes come from sgring::RowAddr::tma.
int make_head_tensor_map(CUtensorMap* out, const void* base, int B, int H, int N, int D, int bnhd, int box_rows,
                         const char* who);

// ---- dense anchored gather (hg_api.cu), shared with the single-gather entry points ----------
// Forward of one anchored gather: anchor A, rows (Rw, Vrow), cols (C, Vcol), all [B,H,N,D] BF16.
int dense_gather_forward(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                         const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int N, int D, int n_valid,
                         cudaStream_t st);
// The same with a length and a valid count per index axis (anchor, rows, cols; valid 0 = all): the three axes of the
// reference's gather (cuda/forward.cu:1436-1452).  A mask needs equal lengths.
struct Axis { int n; int valid; };
int dense_gather_forward_axes(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                              const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int D, Axis a, Axis r,
                              Axis c, cudaStream_t st);
int dense_gather_backward_side_axes(const void* A, const void* dY, const void* Y, const float* m, const float* l,
                                    const void* Ka, const void* Va, const void* Kb, const void* Vb,
                                    const uint8_t* mask, float* dKb, float* dVb, float* dA_part, int B, int H, int D,
                                    Axis a, Axis own, Axis oth, cudaStream_t st, float* chunk_scratch = nullptr);
// Backward for one key side: adds d(Kb), d(Vb) into FP32 planes; if dA_part is non-null also
// accumulates the anchor gradient into one zero-filled partial plane per 128-key tile of the own side.
// chunk_scratch: optional two planes of scratch; with it, short sequences split their anchors over two CTAs
// per (tile, batch, head) and the second CTA's sums are added from there afterwards (fixed order).
int dense_gather_backward_side(const void* A, const void* dY, const void* Y, const float* m, const float* l,
                               const void* Ka, const void* Va, const void* Kb, const void* Vb, const uint8_t* mask,
                               float* dKb, float* dVb, float* dA_part, int B, int H, int N, int D, int n_valid,
                               cudaStream_t st, float* chunk_scratch = nullptr);
int dense_tiles(int N, int n_valid);
int add_planes(const float* src, int n_src, size_t plane, float* acc, cudaStream_t st);
int plane_to_bf16(const float* src, void* out, size_t n, cudaStream_t st);
int dense_status_read_and_clear(int* out);

}  // namespace att3
