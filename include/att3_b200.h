/*
 * att3_b200.h -- C ABI of the sm_100a hypergraph-attention (triplet) kernels.
 *
 * This is the boundary a host binding (pybind, ctypes, cgo, ...) links against:
 * plain device pointers, sizes and a stream, int status codes, no torch types.
 * It replaces the device half of the reference's pybind module
 * att3ntion._cuda_kernels (cpp/cuda_bindings.cpp:30-233, declarations in
 * cpp/cuda_bindings.h:57-156).  The caller owns every buffer: the reference
 * allocates outputs inside its host launchers (cuda/forward.cu:1678-1683); here
 * the binding allocates and passes them in, so nothing in this library calls
 * an allocator.
 *
 * Conventions
 *   - All activations are contiguous BF16, laid out [B, H, N, D]; statistics
 *     m, l are contiguous FP32 [B, H, N].  m is the running maximum of the
 *     scaled score (ATT3_NEG_INF for a query with no visible pair), l the sum
 *     of exp(score - m) (0 for such a query), LSE = m + log(l)
 *     (cpp/cuda_bindings.h:59, cuda/common.cuh:17-24).
 *   - mask, where accepted, is a contiguous byte array [B, N, N] (non-zero =
 *     visible) or NULL.  A pair (j, k) is live for anchor a iff mask[b,a,j] and
 *     mask[b,a,k] (cuda/forward.cu:33-46).
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it
 *     and no entry point synchronises the host.
 *   - Every function returns ATT3_OK or an ATT3_ERR_* code; the message of the
 *     last failure on the calling thread is att3_last_error().
 *   - Pointers must be device pointers valid on the current device.
 */
#ifndef ATT3_B200_H
#define ATT3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATT3_OK 0
#define ATT3_ERR_INVALID 1     /* bad argument: shape, alignment, null pointer, unsupported value */
#define ATT3_ERR_CUDA 2        /* a CUDA runtime call failed; message carries cudaGetErrorString */
#define ATT3_ERR_UNSUPPORTED 3 /* device is not sm_100 or lacks the shared memory the kernel needs */
#define ATT3_ERR_WORKSPACE 4   /* workspace pointer missing or smaller than *_workspace_bytes() */
#define ATT3_ERR_TIMEOUT 5     /* a bounded device-side wait ran out (see att3_device_status) */

#define ATT3_NEG_INF (-1e30f)  /* cuda/common.cuh:24 */

/* Message of the last error raised on this thread ("" if none).  Replaces the
 * TORCH_CHECK exceptions of the reference launchers (cuda/forward.cu:1609-1653). */
const char* att3_last_error(void);

/* ABI revision; bumped when a signature below changes. */
int att3_abi_version(void);

/* Every device-side wait in these kernels (on an mbarrier that a tensor-core
 * commit arrives on) has an iteration limit; a wait that runs out sets a sticky
 * status word on the device and the kernel leaves through its normal exit, so
 * the context stays usable.  This call synchronises `stream`, reads and clears
 * the word of the current device and returns ATT3_OK or ATT3_ERR_TIMEOUT.  The
 * reference has no counterpart (its kernels have no device-side waits). */
int att3_device_status(void* stream);

/* ------------------------------------------------------------------------- *
 * Single query gather:  Y[i] = sum_{j,k} softmax_{j,k}(Q_i.R_j.S_k/sqrt(D)) Vr[j] Vs[k]
 *
 * One pair of entry points covers both reference operators:
 *   Hkv == Hq : single_gather_{forward,backward}_cuda
 *               (cuda/forward.cu:1666-1719, cuda/backward.cu:2248-2353)
 *   Hkv == 1  : single_gather_shared_{forward,backward}_cuda
 *               (cuda/forward.cu:1723-1760, cuda/backward.cu:2512-2582)
 * Q, Y, dY, dQ are [B,Hq,N,D]; R, S, Vr, Vs and their gradients [B,Hkv,N,D].
 * Hq must be a multiple of Hkv; query head h reads KV head h / (Hq/Hkv).
 *
 * window > 0 : equal causal window on both key axes, query i sees keys in
 *              (i - window, i] (cuda/common.cuh:50-85); 1 <= window <= 128.
 *              mask (optional) may only remove keys inside the window.
 * window == 0: every key is a candidate; visibility comes from mask alone
 *              (NULL = all visible).
 * D is 64 or 128 and N a multiple of 16, as in single_gather_check
 * (cuda/forward.cu:1609-1631).
 *
 * q_begin: queries with index < q_begin are not computed (their Y/m/l/dQ rows
 *          are left untouched) but their rows still act as keys.  A rank that
 *          owns query rows [q_begin, N) of a longer sequence passes the
 *          (window-1)-row key halo in front of its rows this way.  0 = all.
 * ------------------------------------------------------------------------- */

/* Scratch bytes att3_sg_backward needs for these sizes (FP32 key-gradient
 * partials that are reduced over heads and query blocks).  Forward needs none. */
size_t att3_sg_backward_workspace_bytes(int B, int Hq, int Hkv, int N, int D, int window);

int att3_sg_forward(const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                    const uint8_t* mask, void* Y, float* m, float* l,
                    int B, int Hq, int Hkv, int N, int D, int window, int q_begin, void* stream);

/* dR, dS, dVr, dVs come back reduced over the query heads of each KV head
 * ([B,Hkv,N,D], one BF16 rounding after the FP32 sum); rows < q_begin of these
 * hold the contributions of this call's queries to the halo keys. */
int att3_sg_backward(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                     const void* Vs, const void* Y, const float* m, const float* l, const uint8_t* mask,
                     void* dQ, void* dR, void* dS, void* dVr, void* dVs,
                     int B, int Hq, int Hkv, int N, int D, int window, int q_begin,
                     void* workspace, size_t workspace_bytes, void* stream);

/* att3_sg_backward with the four key-side gradients left in FP32
 * ([B,Hkv,N,D] floats, same workspace): for a process that holds only part of
 * the query heads of a KV head (heads sharded over GPUs), whose key gradients
 * are partial sums to be added across processes before they are rounded --
 * the reduction the reference performs over its per-head partial buffers inside
 * one GPU (cuda/backward.cu:2548-2575).  Windowed path only (window 1..128). */
int att3_sg_backward_kv32(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                          const void* Vs, const void* Y, const float* m, const float* l,
                          const uint8_t* mask, void* dQ, float* dR, float* dS, float* dVr, float* dVs,
                          int B, int Hq, int Hkv, int N, int D, int window, int q_begin,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Extended calls for the windowed path.  Options beyond the reference's call surface travel in one
 * struct so that the plain entry points keep their signatures; a NULL ext or an all-zero struct is the plain call.
 *   window_s    window on the S / Vs key axis, with `window` then the R / Vr axis's: query i sees the pairs
 *               (j, k) with j in (i - window, i] and k in (i - window_s, i].  0 = equal windows.  The reference
 *               lists independent (W1, W2) windows as an open item (docs/KERNEL_HISTORY.md:180).
 *   mask_words  the caller's mask as packed words [B, N, ceil(N/32)], bit t of word c = key 32 c + t, in place of
 *               the byte mask (pass mask = NULL): the representation of the reference's mask metadata
 *               (cuda/shared_kv/shared_mask_metadata.cuh:8-31), 1/32 of the bytes per query row.
 *   layout      memory layout of Q, R, S, Vr, Vs, Y, dY and all gradients: 0 = [B,H,N,D] contiguous (the
 *               reference's contract, cuda/forward.cu:1609-1631); 1 = [B,N,H,D] contiguous, i.e. the projections'
 *               own output viewed as heads -- the reference's module permutes and copies every operand into
 *               layout 0 on every call (att3ntion/_autograd.py:349-363), which this removes.  m, l stay [B,H,N].
 *   Y_act       forward only: a second output QuickGELU(Y) = Y * sigmoid(1.702 Y), laid out like Y (the module's
 *               activation, att3ntion/_autograd.py:254-256, written from the forward's epilogue), or NULL.
 *   precise     1: the score product runs on the Hadamard operand split into its BF16 value and the exact BF16
 *               residual (two tensor-core products instead of one), so the scores carry no rounding of Q o R; the
 *               reference prototyped this "compensated" path for its stress gates and did not ship it
 *               (docs/KERNEL_HISTORY.md:22, 185).  Forward and backward must use the same setting.  Always the
 *               128-slot ring schedule; 1.8x the time of the plain call at the headline shape (27.0 against 14.9 ms).
 * All need window >= 1.  att3_sg_pack_mask produces the words (and, optionally, the per-query count of
 * visible keys inside the causal window saturated at 2, [B, N] bytes; window = 0: the mask alone). */
typedef struct att3_sg_ext {
    int window_s;
    const uint32_t* mask_words;
    int layout;
    void* Y_act;
    int precise;
} att3_sg_ext;

int att3_sg_forward_ext(const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                        const uint8_t* mask, void* Y, float* m, float* l,
                        int B, int Hq, int Hkv, int N, int D, int window, int q_begin, void* stream,
                        const att3_sg_ext* ext);
int att3_sg_backward_ext(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                         const void* Vs, const void* Y, const float* m, const float* l, const uint8_t* mask,
                         void* dQ, void* dR, void* dS, void* dVr, void* dVs,
                         int B, int Hq, int Hkv, int N, int D, int window, int q_begin,
                         void* workspace, size_t workspace_bytes, void* stream, const att3_sg_ext* ext);
int att3_sg_pack_mask(const uint8_t* mask, uint32_t* words, uint8_t* support, int B, int N, int window, void* stream);

/* One key side of att3_sg_backward_kv32 per call: side 0 writes dQ, dS, dVs
 * (the other gradient pointers may be NULL), side 1 writes dR, dVr.  Two calls,
 * side 0 then side 1, equal one att3_sg_backward_kv32 bit for bit; in between a
 * multi-GPU caller can start summing the first side's partials across
 * processes while the second side is computed (the reference reduces its
 * per-head partials only after all passes, cuda/backward.cu:2558-2575). */
int att3_sg_backward_kv32_side(int side, const void* dY, const void* Q, const void* R, const void* S,
                               const void* Vr, const void* Vs, const void* Y, const float* m, const float* l,
                               const uint8_t* mask, void* dQ, float* dR, float* dS, float* dVr, float* dVs,
                               int B, int Hq, int Hkv, int N, int D, int window, int q_begin,
                               void* workspace, size_t workspace_bytes, void* stream);

/* att3_sg_backward for callers that cannot allocate device memory.  It has no
 * counterpart in the reference, whose launchers allocate their own buffers
 * through torch.  Meant for hosts where an allocator call is impossible or
 * forbidden at the point of the call: code running inside a framework's
 * capture-private or stream-ordered pool, a real-time loop with a fixed memory
 * plan, a sandboxed worker without access to the allocation entry points.
 * The FP32 scratch of the windowed backward lives in a fixed array inside the
 * library (att3_sg_backward_static_max_bytes(), 32 MiB, held by every GPU that
 * loads the library until the process exits), so the call itself allocates
 * nothing: no cudaMalloc/cudaFree, no allocating library routine (leave
 * att3_timing_enable off, it creates events).
 *   - windowed path only (1 <= window <= 128); sizes whose scratch
 *     (att3_sg_backward_workspace_bytes: 16 * B * Hkv * N * D bytes when the
 *     query blocks are at least 127 long, more for shorter blocks) exceeds the
 *     array are rejected with ATT3_ERR_WORKSPACE and a message naming both;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it: make that
 *     first call before any stream capture;
 *   - all calls share the one array and it keeps the last call's contents;
 *     nothing in it needs clearing between calls, but two calls that can overlap
 *     on the GPU (different streams) race on it -- serialise them;
 *   - results are bit-identical to att3_sg_backward on the same inputs. */
size_t att3_sg_backward_static_max_bytes(void);
int att3_sg_backward_static(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                            const void* Vs, const void* Y, const float* m, const float* l, const uint8_t* mask,
                            void* dQ, void* dR, void* dS, void* dVr, void* dVs,
                            int B, int Hq, int Hkv, int N, int D, int window, int q_begin, void* stream);

/* ------------------------------------------------------------------------- *
 * Three-gather hypergraph attention: forward_cuda / backward_cuda
 * (cuda/forward.cu:1252-1602, cuda/backward.cu:1716-2232; math in
 * cpp/torch_reference.cpp:24-57).  All nine inputs are [B,H,N,D] with
 * D in {16,32,64,128}.  Outputs Y_q, Y_r, Y_s (gathers) and Y_q_, Y_r_, Y_s_
 * (scatters, cuda/forward.cu:941-1249; computed when scatter != 0, else zero-filled) are BF16
 * [B,H,N,D]; the six statistics FP32 [B,H,N].  n_valid < N marks trailing
 * padding rows that are invisible in every role (0 or N: none).  gather_mode 1
 * computes only the Q-anchored gather; the other outputs are zero-filled and
 * their statistics set to (m = +1e30, l = 1) as the reference does
 * (cuda/forward.cu:1455-1459).
 * ------------------------------------------------------------------------- */
int att3_hg_forward(const void* Q, const void* R, const void* S,
                    const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2,
                    const void* Vs1, const void* Vs2, const uint8_t* mask,
                    void* Yq, void* Yr, void* Ys, void* Yq_, void* Yr_, void* Ys_,
                    float* m_i, float* l_i, float* m_j, float* l_j, float* m_k, float* l_k,
                    int B, int H, int N, int D, int n_valid, int gather_mode, int scatter, void* stream);

size_t att3_hg_backward_workspace_bytes(int B, int H, int N, int D);

/* Nine gradients (Q,R,S,Vq1,Vq2,Vr1,Vr2,Vs1,Vs2), BF16 [B,H,N,D].  g* are the
 * cotangents of the six outputs; pass scatter = 0 when the three scatter
 * cotangents are identically zero (att3ntion/_custom_op.py:73-96), scatter = 1
 * adds the gradients of the scatter outputs (cuda/backward.cu:175-316, 949-1613;
 * gather_mode 0 only; the same tensor-core kernels in their scatter forms,
 * fixed summation order).  Yq, Yr, Ys
 * are the forward's gather outputs: the softmax Jacobian correction is taken as
 * rowsum(dY o Y), the reference's tensor-core path (cuda/backward.cu:1835-1837).
 * With gather_mode 1 only the Q-anchored tensors are read. */
int att3_hg_backward(const void* gYq, const void* gYr, const void* gYs,
                     const void* gYq_, const void* gYr_, const void* gYs_,
                     const void* Q, const void* R, const void* S,
                     const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2,
                     const void* Vs1, const void* Vs2,
                     const void* Yq, const void* Yr, const void* Ys,
                     const float* m_i, const float* l_i, const float* m_j, const float* l_j,
                     const float* m_k, const float* l_k, const uint8_t* mask,
                     void* dQ, void* dR, void* dS, void* dVq1, void* dVq2, void* dVr1, void* dVr2,
                     void* dVs1, void* dVs2,
                     int B, int H, int N, int D, int n_valid, int gather_mode, int scatter,
                     void* workspace, size_t workspace_bytes, void* stream);

/* The same operator with a length per axis: Q, Vq*, Yq*, dQ ... are [B,H,I,D], the R tensors [B,H,J,D], the S
 * tensors [B,H,K,D], the statistics [B,H,I], [B,H,J], [B,H,K] (cuda/forward.cu:1281-1285), and I_valid, J_valid,
 * K_valid mark trailing padding per axis (cuda/forward.cu:1300-1302, cpp/cuda_bindings.cpp:143-177: each defaults
 * to its length when <= 0 or larger).  As in the reference, a mask and the scatter outputs need I == J == K
 * (cuda/forward.cu:1292, 1545); the scatter outputs also take one valid length for all three axes.  The reference's
 * backward has no valid lengths (cpp/cuda_bindings.cpp:179-205: padded slots take part); the ones given here are
 * applied like the forward's, pass zeros for the reference's behaviour.
 * att3_hg_forward / att3_hg_backward are these with I = J = K = N and one valid length. */
int att3_hg_forward_axes(const void* Q, const void* R, const void* S,
                         const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2,
                         const void* Vs1, const void* Vs2, const uint8_t* mask,
                         void* Yq, void* Yr, void* Ys, void* Yq_, void* Yr_, void* Ys_,
                         float* m_i, float* l_i, float* m_j, float* l_j, float* m_k, float* l_k,
                         int B, int H, int I, int J, int K, int D, int I_valid, int J_valid, int K_valid,
                         int gather_mode, int scatter, void* stream);

size_t att3_hg_backward_axes_workspace_bytes(int B, int H, int I, int J, int K, int D);

int att3_hg_backward_axes(const void* gYq, const void* gYr, const void* gYs,
                          const void* gYq_, const void* gYr_, const void* gYs_,
                          const void* Q, const void* R, const void* S,
                          const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2,
                          const void* Vs1, const void* Vs2,
                          const void* Yq, const void* Yr, const void* Ys,
                          const float* m_i, const float* l_i, const float* m_j, const float* l_j,
                          const float* m_k, const float* l_k, const uint8_t* mask,
                          void* dQ, void* dR, void* dS, void* dVq1, void* dVq2, void* dVr1, void* dVr2,
                          void* dVs1, void* dVs2,
                          int B, int H, int I, int J, int K, int D, int I_valid, int J_valid, int K_valid,
                          int gather_mode, int scatter, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- *
 * Host-side helpers (no GPU needed).
 * ------------------------------------------------------------------------- */

/* Window -> visited tile ranges, the contract of sg_row_bounds / sg_col_bounds
 * (cuda/common.cuh:50-85) that the reference exposes as sg_tile_ranges
 * (cpp/cuda_bindings.cpp:117-132).  side 0: the query is anchor a; side 1: a is
 * a key and the queries are the rows.  Writes up to max_out (j0, k_lo, k_hi)
 * triples into out[3*i..] and returns the number of row blocks (or -1 on a bad
 * argument). */
int att3_sg_tile_ranges(int N, int window, int a, int side, int bj, int bk, int* out, int max_out);

/* Packs up to 32 mask bytes into one word, bit t = (row[t] != 0); never reads
 * outside [row, row+lim).  Contract of sg_pack_mask32 (cuda/common.cuh:87-101). */
uint32_t att3_pack_mask32(const uint8_t* row, int lim);

/* Query-block partition the windowed kernels use: number of CTAs launched and
 * queries per block for these sizes on a device with `sm_count` SMs. */
int att3_sg_query_blocks(int B, int Hq, int Hkv, int N, int q_begin, int sm_count, int* block_len);

/* Schedule override, the counterpart of the reference's tile overrides (SgConfig,
 * cpp/cuda_bindings.h:18-48; sg_set_config, cpp/cuda_bindings.cpp:88-106): queries
 * per CTA of the windowed forward and of the windowed backward passes; 0 restores
 * the built-in choice, other values must be >= 16.  Process-wide.  The backward's
 * workspace size depends on its block length (shorter blocks need more partial
 * planes): query att3_sg_backward_workspace_bytes after changing it. */
int att3_sg_set_query_block(int fwd_len, int bwd_len);

/* Windows of at most 64 keys run a schedule that packs 128 / W queries into one tensor-core tile (D = 128,
 * at least four query heads per KV head, q_begin a multiple of 8); everything else runs the 128-slot ring
 * schedule.  on = 0 sends every windowed call to the ring schedule (the counterpart of fwd_group / rs_group
 * selecting a fixed schedule in the reference, cuda/forward.cu:1739, cuda/backward.cu:2518-2525).  Returns the
 * previous setting.  Process-wide. */
int att3_sg_set_packed(int on);

/* Launch counters, the counterpart of att3_tc::State (cpp/cuda_bindings.h:18-48).
 * which: 0 single-gather forward, 1 single-gather backward, 2 three-gather
 * forward, 3 three-gather backward.  Returns kernels launched so far. */
unsigned long long att3_launch_count(int which);

/* Per-kernel device timing for benchmarks (no counterpart in the reference,
 * which times whole calls from Python: benchmarks/bench_single_gather.py:965-982).
 * While enabled, every kernel launch is bracketed by CUDA events on its own
 * stream.  att3_timing_read waits for the recorded launches of one kernel,
 * returns their summed duration and count, and forgets them.  kernel_id:
 * 0 windowed forward, 1 windowed backward pass, 2 key-gradient reduction,
 * 3 dense forward, 4 dense backward, 5 three-gather helpers.
 * att3_timing_enable returns the previous setting. */
int att3_timing_enable(int on);
int att3_timing_read(int kernel_id, double* total_ms, unsigned long long* launches);

/* ------------------------------------------------------------------------- *
 * Self-tests (no counterpart in the reference, whose kernels have neither
 * operand descriptors nor device-side waits).
 *
 * att3_umma_selftest multiplies two 128x128 BF16 matrices on one CTA through
 * the operand arrangement `mode` selects and writes the FP32 product to D
 * (row-major [128][128]); the shared-memory descriptor encodings are the fixed
 * ones the kernels use.
 *   mode 0: D = A B^T   (A and B K-major in shared memory)
 *   mode 1: D = A B     (A K-major, B MN-major)
 *   mode 2: D = A^T B   (A and B MN-major)
 *   mode 3: D = A B     (A in tensor memory, B MN-major)
 *   mode 4: D = A B^T   (A in tensor memory, B K-major)
 *   mode | 8: issued as an N = 64 instruction; only the first 64 columns of D are written.
 * status_dev[0] receives 1 if the bounded wait for the product ran out.
 *
 * att3_wait_selftest launches a kernel in which one thread waits, for at most
 * `limit` polls, on a barrier that nothing arrives on.  The wait gives up, the
 * kernel records that in the device status word and returns normally; the next
 * att3_device_status() on that device reports ATT3_ERR_TIMEOUT and clears the
 * word.  This is the whole failure path of the kernels' bounded waits, driven
 * without a fault or a hang.
 * ------------------------------------------------------------------------- */
int att3_umma_selftest(const void* A, const void* B, float* D, int mode, int* status_dev, void* stream);
int att3_wait_selftest(unsigned limit, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATT3_B200_H */
