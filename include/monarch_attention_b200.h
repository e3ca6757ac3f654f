/*
 * monarch_attention_b200 - C ABI of the B200 (sm_100a) MonarchAttention forward library.
 *
 * This is the boundary a binding of the reference's attention module links against.
 * Every entry point takes plain pointers, sizes and a stream handle; no framework types.
 *
 * What it replaces in the reference:
 *   - an implementation function as registered with the module
 *     (reference: ma/monarch_attention.py:11-19, signature
 *      fn(q, k, v, attn_mask | None, T, B, pre_pad) -> Tensor), i.e.
 *     monarch_attention_torch (reference: ma/ma_torch.py:65-108) and
 *     monarch_attention_triton (reference: ma/ma_triton.py:641-788);
 *   - the four stage functions that call evaluates
 *     (reference: ma/ma_torch.py:10-23, :26-35, :38-52, :55-62).
 *
 * Memory ownership: the caller owns q, k, v, out, mask and the workspace (all device
 * memory of the current device).  The library allocates no device memory in
 * ma_b200_forward.  Work is enqueued on the given stream and is stream-ordered.
 *
 * Tensors are 4-D views (E, H, N, W) whose innermost stride is 1 element; the other
 * three strides are arbitrary element strides (so a permuted (E, N, H, W) buffer is
 * accepted without a copy).
 */
#ifndef MONARCH_ATTENTION_B200_H_
#define MONARCH_ATTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MA_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define MA_B200_API __attribute__((visibility("default")))
#else
#define MA_B200_API
#endif

/* Return codes of every entry point that returns int. */
enum {
  MA_B200_OK = 0,
  MA_B200_INVALID_ARGUMENT = 1, /* NULL pointer, bad shape / stride / alignment / dtype       */
  MA_B200_UNSUPPORTED = 2,      /* valid problem that the requested kernel cannot run         */
  MA_B200_CUDA_ERROR = 3,       /* a CUDA runtime / driver call failed (see last_error)       */
  MA_B200_DEVICE_WAIT_EXPIRED = 4, /* a bounded on-device wait gave up; output is undefined   */
  MA_B200_WORKSPACE_TOO_SMALL = 5
};

/* Element types.  q and k share qk_dtype; v and out share v_dtype. */
enum { MA_B200_F32 = 0, MA_B200_BF16 = 1, MA_B200_F16 = 2 };

/* Kernel families.  AUTO picks the fused tcgen05 kernel when the problem fits it, else the
 * warp-level tensor-core kernels, else the generic kernels.
 *   GENERIC        SIMT stage kernels, any shape / dtype / mask (2T launches)
 *   TCGEN05        persistent tcgen05 kernel, all 2T stages in one launch: 16-bit inputs,
 *                  D = Dv = 64, no mask, no padding, block size = block count = 128 or 64
 *   TCGEN05_STAGED the same kernel launched once per stage (for per-stage timing)
 *   WARP_MMA       warp-level tensor-core stage kernels for 16-bit inputs with block size and
 *                  block count up to 256 and D <= 80 (D <= 64 when either exceeds 128)
 *                  (2T launches; masks and padding handled)
 *   HEAD_FUSED     one CTA per head, one iteration (T = 1), block size and count <= 32, D <= 64,
 *                  the head's Q, K, V, al and y together within 227 KB of shared memory: both
 *                  stages in one launch, HBM sees Q, K, V once and the result once (1 launch) */
enum {
  MA_B200_KERNEL_AUTO = 0,
  MA_B200_KERNEL_GENERIC = 1,
  MA_B200_KERNEL_TCGEN05 = 2,
  MA_B200_KERNEL_TCGEN05_STAGED = 3, /* (4 is not in use) */
  MA_B200_KERNEL_WARP_MMA = 5,
  MA_B200_KERNEL_HEAD_FUSED = 6
};

typedef struct ma_b200_tensor {
  void* ptr;        /* device pointer to element (0,0,0,0)            */
  int64_t stride_e; /* element strides; the innermost stride is 1     */
  int64_t stride_h;
  int64_t stride_n;
} ma_b200_tensor;

/*
 * One forward call.  Field meaning follows the reference's implementation-function
 * arguments (reference: ma/ma_torch.py:65-73): num_steps = T, block_size = B,
 * pre_pad != 0 pads the token axis at the front.  mask is the (E, N) key/query
 * validity mask, one byte per token, non-zero = valid, or NULL
 * (reference: ma/ma_torch.py:96-98 combines it with the padding mask).
 */
typedef struct ma_b200_problem {
  int32_t abi_version; /* MA_B200_ABI_VERSION */
  int32_t E, H, N, D, Dv;
  int32_t block_size;
  int32_t num_steps;
  int32_t pre_pad;
  int32_t qk_dtype;
  int32_t v_dtype;
  int32_t kernel; /* MA_B200_KERNEL_* */
  ma_b200_tensor q, k, v, out;
  const uint8_t* mask;
  int64_t mask_stride_e;
} ma_b200_problem;

/* Byte offsets of the stage-to-stage state inside the workspace (for tests and tools).
 * ar: (E*H, M, B, D) qk_dtype   cr: (E*H, M, B) f32
 * al: (E*H, B, M, D) qk_dtype   cl: (E*H, B, M) f32   y: (E*H, B, M, Dv) v_dtype
 * status: one int32 device flag, 0 = no device-side error.
 * counters: (E*H, 2T) int32 stage-completion counters of the fused kernel. */
typedef struct ma_b200_workspace_layout {
  size_t status, counters, ar, cr, al, cl, y, total;
  int32_t M;
  int32_t kernel; /* the family AUTO resolves to */
} ma_b200_workspace_layout;

/* Scratch bytes ma_b200_forward needs for this problem (0 on an invalid problem).
 * The workspace must be 256-byte aligned.
 * reference: the Triton launcher allocates the same state per call (ma/ma_triton.py:669-676,734). */
MA_B200_API size_t ma_b200_workspace_bytes(const ma_b200_problem* p);

/* Fill *layout; returns MA_B200_OK or an error code. */
MA_B200_API int ma_b200_workspace_layout_of(const ma_b200_problem* p, ma_b200_workspace_layout* layout);

/* Enqueue the forward pass on `stream` (a cudaStream_t / CUstream; NULL = default stream).
 * reference: monarch_attention_torch, ma/ma_torch.py:65-108. */
MA_B200_API int ma_b200_forward(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream);

/* Same as ma_b200_forward, and additionally records one CUDA event pair per stage launch
 * and, after synchronising the stream, writes the stage durations in milliseconds to
 * stage_ms[0 .. min(n_stage_ms, 2*num_steps) - 1] in launch order (the fused kernel has a single
 * launch: its duration is stage_ms[0], the other entries are 0).  Blocks the host.
 * reference: the per-kernel NVTX/ncu harness, perfbench/bench.py:199-223. */
MA_B200_API int ma_b200_forward_timed(const ma_b200_problem* p, void* workspace, size_t workspace_bytes, void* stream,
                          float* stage_ms, int32_t n_stage_ms);

/* Synchronise `stream` and read the device-side status flag of the last forward that used
 * this workspace: MA_B200_OK or MA_B200_DEVICE_WAIT_EXPIRED. */
MA_B200_API int ma_b200_device_status(void* workspace, void* stream);

/* Without synchronising anything: has a bounded wait of the fused tcgen05 kernel given up on `device`
 * since the last poll?  A CTA that gives up stores its code in a page-locked host word the library
 * maps once per device (at the first fused launch there), so the answer trails the GPU by at most
 * the kernels still in flight.  MA_B200_OK, or MA_B200_DEVICE_WAIT_EXPIRED once per incident (the
 * word is cleared by the poll).  This is the lazily read error flag of the eager call: the reference
 * raises from inside the call (ma/monarch_attention.py:50-59), an asynchronous launch cannot.
 * No counterpart in the reference. */
MA_B200_API int ma_b200_poll_device_status(int device);

/* Self-test of the give-up path (no counterpart in the reference): launches the left-factor stage of
 * `p` (num_steps >= 2, a problem the fused kernel takes) alone, with the completion counters it waits
 * on left at zero and a short patience, so that every CTA's bounded wait runs out and the kernel
 * returns by itself after a few hundred microseconds.  Afterwards ma_b200_device_status(workspace)
 * and ma_b200_poll_device_status() report MA_B200_DEVICE_WAIT_EXPIRED, and the next ordinary call is
 * unaffected.  Nothing faults, traps or spins without bound. */
MA_B200_API int ma_b200_selftest_wait_expiry(const ma_b200_problem* p, void* workspace, size_t workspace_bytes,
                                             void* stream);

/* Test hook (no counterpart in the reference): with on != 0 the generic kernel family always runs its
 * general warp-per-row form, also on tiles of up to 16 x 16 where it would take the thread-per-logit
 * form.  The two forms are meant to return the same bits; tests/test_parity_gpu.py holds them to that.
 * Process-wide; 0 restores the default. */
MA_B200_API void ma_b200_selftest_generic_general_form(int on);

/* Human-readable text for a return code. */
MA_B200_API const char* ma_b200_status_string(int status);

/* Detail of the last failure on the calling thread ("" if none). */
MA_B200_API const char* ma_b200_last_error(void);

/*
 * Forward pass for callers that cannot allocate device memory (no counterpart in the
 * reference, which allocates its state per call).
 *
 * Who needs it: a host process that gave all device memory to its own pool at start-up, a
 * plug-in that must not call the CUDA allocator, a latency-critical loop where an allocator
 * call is not acceptable.  Such a caller cannot supply the workspace ma_b200_forward wants.
 * Here the stage-to-stage state lives in a fixed array inside the library image:
 * MA_B200_STATIC_SCRATCH_BYTES on every GPU that loads the library, held until the process
 * exits.  The caller passes q, k, v, out and mask exactly as for ma_b200_forward; p->kernel
 * is ignored and the generic kernel family runs.  Nothing is allocated or freed, on the
 * device or through any allocating library call.
 *
 * Limits and rules:
 *  - a problem whose state (ma_b200_workspace_bytes with kernel = GENERIC) exceeds
 *    MA_B200_STATIC_SCRATCH_BYTES is refused with MA_B200_WORKSPACE_TOO_SMALL;
 *  - the first call on each device looks up the device address of the array (with that
 *    device current) and caches it; make that first call before any stream capture begins;
 *  - all calls on one GPU share the one array, which keeps the previous call's contents
 *    (the library clears the one word that must start at zero): calls that may overlap in
 *    time on the GPU - different streams, different host threads - race on it and must be
 *    serialised by the caller; calls queued on a single stream are safe.
 * Failure detail: ma_b200_static_scratch_last_error().
 */
#define MA_B200_STATIC_SCRATCH_BYTES ((size_t)8 << 20)
MA_B200_API int ma_b200_forward_static_scratch(const ma_b200_problem* p, void* stream);
MA_B200_API size_t ma_b200_static_scratch_bytes(void);
MA_B200_API const char* ma_b200_static_scratch_last_error(void);

/* Library ABI version (MA_B200_ABI_VERSION at build time). */
/*
 * Forward pass for q, k, v and the result in HOST memory, PCIe copies overlapped with the
 * kernels.  No counterpart in the reference, whose module is handed device tensors
 * (reference: ma/monarch_attention.py:50-59) and leaves the copies to its caller.
 *
 * p->q, k, v, out (and p->mask) are HOST pointers with the usual element strides; page-locked
 * memory is needed for the copies to overlap, pageable memory works but serialises.  The
 * (batch, head) pairs are processed in chunks of heads_per_chunk heads (smaller ones at the very
 * end, so that little work is left once the last copy-in has landed): H2D of chunk i+1,
 * ma_b200_forward on chunk i and D2H of chunk i-1 run on three streams owned by the library,
 * with three staging slots and the chunk workspace in device_scratch (256-byte aligned, at
 * least ma_b200_host_scratch_bytes(p, heads_per_chunk) bytes; 0 = invalid problem).
 * The call only queues work: it is ordered after what is already queued on `stream`, and on
 * return `stream` has been made to wait for the last kernel and the last copy, so the result
 * is in p->out once `stream` has been synchronised.  Calls on one device share the library's
 * streams and events and must not overlap in time (one host thread, one caller stream, or
 * explicit ordering by the caller).  Failure detail: ma_b200_host_last_error().
 */
MA_B200_API size_t ma_b200_host_scratch_bytes(const ma_b200_problem* p, int heads_per_chunk);
MA_B200_API int ma_b200_forward_host(const ma_b200_problem* p, int heads_per_chunk, void* device_scratch,
                                     size_t scratch_bytes, void* stream);
/* The same for a stream of calls (no counterpart in the reference).  The host buffers of q, k, v (and the
 * mask) must be valid when the call is made - nothing queued on `stream` is waited for before the copy-in
 * starts - and when the previous call on this device used the same scratch with the same layout, this call's
 * copy-in runs while that call's kernels and copy-out are still in flight, so that back-to-back calls keep
 * the host-to-device link busy all the time.  `stream` is made to wait for this call's last kernel and last
 * copy, as above; results arrive in call order. */
MA_B200_API int ma_b200_forward_host_streamed(const ma_b200_problem* p, int heads_per_chunk, void* device_scratch,
                                              size_t scratch_bytes, void* stream);
MA_B200_API const char* ma_b200_host_last_error(void);

MA_B200_API int32_t ma_b200_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MONARCH_ATTENTION_B200_H_ */
