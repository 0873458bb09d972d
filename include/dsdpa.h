/*
 * dsdpa.h -- C ABI of the B200 (sm_100a) fused deformable multi-head
 * scaled-dot-product attention library (libdeform_sdpa.so).
 *
 * The library replaces the device side of the reference's fused operator:
 * the Triton kernels _fwd_kernel (ops/triton.py:27-194), _bwd_preprocess
 * (ops/triton.py:197-215) and _bwd_kernel (ops/triton.py:219-365), and the tensor
 * passes the operator's host code runs around them (coordinate scaling,
 * zero fills, K pre-scaling and dtype casts, ops/triton.py:381-383, 389,
 * 427-432, 461-462).  Results follow the reference's pure-PyTorch path
 * (ops/torch.py:5-28): bilinear sampling with align_corners=True and zero padding
 * per corner.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer of the device passed in `device`, 16-byte
 *     aligned, to a contiguous tensor.  The library borrows them for the duration of
 *     the enqueued work and never allocates or frees memory.
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL
 *     is the legacy default stream) and returns a dsdpa_status.  No call throws,
 *     aborts or synchronises the device, except dsdpa_device_error().
 *   - Tensor layouts are the reference's (README.md:35-38):
 *       q, k, v, out, dout, dq, dk, dv : [B, V, Hh, L, D]   L = W*H, pixel (x,y) = y*W+x
 *       coords                         : [B, V, L, V, S, 2] fp32, (x, y) normalised to [0,1]
 *       lse                            : [B, V, Hh, L]      fp32, base-2 log-sum-exp
 */
#ifndef DSDPA_H_
#define DSDPA_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSDPA_VERSION 100

typedef enum dsdpa_status {
    DSDPA_OK = 0,
    DSDPA_ERR_NULL_POINTER = 1,
    DSDPA_ERR_BAD_DTYPE = 2,       /* the reference raises NotImplementedError (ops/triton.py:375) */
    DSDPA_ERR_BAD_HEAD_DIM = 3,    /* the reference asserts D in {16,32,64,128,256} (ops/triton.py:386) */
    DSDPA_ERR_BAD_SHAPE = 4,       /* a non-positive extent, or more elements than the index type holds */
    DSDPA_ERR_MISALIGNED = 5,      /* a pointer that is not 16-byte aligned */
    DSDPA_ERR_WORKSPACE = 6,       /* workspace missing or smaller than dsdpa_backward_workspace_bytes */
    DSDPA_ERR_BAD_FLAGS = 7,
    DSDPA_ERR_CUDA = 8,            /* a CUDA runtime call failed; see dsdpa_last_cuda_error() */
    DSDPA_ERR_DEVICE_TIMEOUT = 9,  /* a bounded wait inside a kernel gave up (dsdpa_device_error) */
    DSDPA_ERR_TOO_LARGE = 10,      /* beyond a stated maximum of the entry point */
    DSDPA_ERR_PEER_ACCESS = 11,    /* a mirror lies in memory the launching device cannot store to */
    DSDPA_ERR_DEVICE_BOUNDS = 12   /* checked build only: a kernel computed an index out of range and
                                      skipped the access (dsdpa_device_error) */
} dsdpa_status;

typedef enum dsdpa_dtype {
    DSDPA_F32 = 0,
    DSDPA_BF16 = 1,
    DSDPA_F16 = 2
} dsdpa_dtype;

/* Flags (OR-ed).  0 selects the default path for the shape. */
#define DSDPA_FLAG_MAPS_FROM_L2    0x1u /* never stage K/V maps in shared memory: gather with read-only loads */
#define DSDPA_FLAG_DETERMINISTIC   0x2u /* backward: two-pass dK/dV with a fixed summation order: dq, dk, dv
                                           are bit-reproducible run to run (the default form where the
                                           shape allows it; the flag refuses the scatter flags).  dcoords,
                                           summed over the heads with floating-point reductions, is not */
#define DSDPA_FLAG_SCATTER_GLOBAL  0x4u /* backward scatter: reductions straight to global memory,
                                           no shared-memory privatised accumulation */
#define DSDPA_FLAG_SCATTER         0x8u /* backward: force the one-kernel scatter form */
#define DSDPA_FLAG_ROUNDED_WEIGHTS 0x10u /* forward, 16-bit storage only (no effect on fp32): the weights
                                           p*w_c that multiply the V rows are rounded to the storage type
                                           first -- what casting P to bf16 before P.V is in dense attention
                                           kernels -- so that V rows are never unpacked to fp32.  Products
                                           stay exact and sums fp32; the reference keeps these weights in
                                           fp32 (ops/triton.py:178), and so does the default */

/* Problem description shared by all entry points. */
typedef struct dsdpa_problem {
    int B;          /* batch */
    int V;          /* views (query views == key views) */
    int Hh;         /* attention heads */
    int W, H;       /* feature-map width and height; L = W*H pixels */
    int D;          /* head dimension, one of 16, 32, 64, 128, 256 */
    int S;          /* sampling points per (query, key view) */
    float sm_scale; /* softmax scale applied to q.k */
    int dtype;      /* dsdpa_dtype of q, k, v, out, dout, dq, dk, dv */
    unsigned flags; /* DSDPA_FLAG_* */
} dsdpa_problem;

/*
 * Forward.  Replaces _fused_deform_sdpa.forward's device work (ops/triton.py:379-416):
 * writes out (storage dtype) and lse (what the reference calls M, ops/triton.py:187-190).
 */
int dsdpa_forward(const dsdpa_problem* p,
                  const void* q, const void* k, const void* v, const float* coords,
                  void* out, float* lse, int device, void* stream);

/*
 * Bytes of scratch dsdpa_backward needs for this problem (0 is possible).
 * Depends on the shape, dtype and flags only.  Two-pass form: fp32 accumulator maps (four times
 * the element count of dk for 16-bit storage, twice for fp32), 8 bytes per (query-head, sample)
 * of first-pass scalars and the sorted index (about 32 bytes per (query, sample), shared by the
 * heads); roughly 3.5x the bytes of q, k, v, out, dout, dq, dk, dv together at the scaling
 * configuration.  The reference allocates its fp32 dK/dV accumulators per call as well
 * (ops/triton.py:427-430).
 */
size_t dsdpa_backward_workspace_bytes(const dsdpa_problem* p);

/*
 * 1 if dsdpa_backward can produce the coordinate gradient (its `dcoords` argument) for this
 * problem, 0 if not: the gradient is computed by the two-pass form only, and problems that form
 * cannot take (a map too large for its index builder, or the scatter flags) are refused with
 * DSDPA_ERR_BAD_FLAGS when dcoords is given.  The reference never returns this gradient
 * (ops/triton.py:464 returns None for coords); callers that may not get it ask here first.
 */
int dsdpa_backward_supports_dcoords(const dsdpa_problem* p);

/*
 * Backward.  Replaces _fused_deform_sdpa.backward's device work (ops/triton.py:419-464):
 * delta = sum(out*dout) (ops/triton.py:197-215), dq (ops/triton.py:339, 362-365) and the
 * dK/dV scatter (ops/triton.py:342-360), including the zero fill of the accumulators and
 * the cast to the storage dtype.  dq, dk, dv are overwritten.
 * dcoords may be NULL (the reference returns no coordinate gradient, ops/triton.py:464);
 * when given it receives d(loss)/d(coords), fp32, same shape as coords.
 */
int dsdpa_backward(const dsdpa_problem* p,
                   const void* q, const void* k, const void* v, const float* coords,
                   const void* out, const float* lse, const void* dout,
                   void* dq, void* dk, void* dv, float* dcoords,
                   void* workspace, size_t workspace_bytes, int device, void* stream);

/*
 * Results stored twice.  (No counterpart in the reference, which runs on one GPU; this is the
 * partitioner's final gather, ops/triton.py has nothing after its kernels, folded into them.)
 *
 * A mirror is a second destination with the layout of the result it shadows.  It may lie in
 * another GPU's memory that is mapped into this process (CUDA IPC, cuMemMap, a peer-enabled
 * cudaMalloc): the kernels that produce a result store each row to both places with plain
 * 16-byte stores, so the transfer to the device that collects a sharded job's results is spread
 * over the kernels' run time instead of following them as a collective.  Mirrors are only
 * written, never read.  Any member (or the whole struct pointer) may be NULL; a mirror must be
 * 16-byte aligned and must not alias an input or a result of the same call.
 * Before anything is launched every mirror is looked up (cudaPointerGetAttributes): for one
 * that lies on another device, peer access from `device` to that device is switched on if it is
 * not yet (cudaDeviceEnablePeerAccess; it stays on), and a mirror `device` cannot reach is
 * refused with DSDPA_ERR_PEER_ACCESS.  (Memory mapped with cuMemMap follows cuMemSetAccess
 * instead: the caller grants `device` write access to it.)
 *
 *   out: written by dsdpa_forward_mirrored; by dsdpa_backward_mirrored it is filled with a copy of
 *        the `out` INPUT (the first pass reads those rows anyway), so that a forward + backward
 *        step sends everything from the backward.
 *   dq, dk, dv: written by dsdpa_backward_mirrored.
 */
typedef struct dsdpa_mirrors {
    void* out;
    void* dq;
    void* dk;
    void* dv;
} dsdpa_mirrors;

int dsdpa_forward_mirrored(const dsdpa_problem* p,
                           const void* q, const void* k, const void* v, const float* coords,
                           void* out, float* lse, void* out_mirror, int device, void* stream);

int dsdpa_backward_mirrored(const dsdpa_problem* p,
                            const void* q, const void* k, const void* v, const float* coords,
                            const void* out, const float* lse, const void* dout,
                            void* dq, void* dk, void* dv, float* dcoords,
                            void* workspace, size_t workspace_bytes,
                            const dsdpa_mirrors* mirrors, int device, void* stream);

/*
 * Sharing a mirror's memory between the processes of one machine (CUDA IPC; plumbing for the
 * mirrors above, no counterpart in the reference).  Nothing is allocated or freed.
 *
 *   dsdpa_peer_export  (owner process) describes the cudaMalloc'd block that holds `ptr`:
 *       a 64-byte handle of the whole block and the offset of `ptr` inside it.  Send both to
 *       the other processes by any means.
 *   dsdpa_peer_import  (other process) maps the block into THIS process for kernels launched on
 *       `device` -- the mapping is made with `device` current and peer access to the owner's GPU
 *       is switched on, which a mapping made under another device does not give -- and returns
 *       the address that corresponds to `ptr`.  Import a block once per process: hand out
 *       sub-ranges yourself.
 *   dsdpa_peer_release unmaps what dsdpa_peer_import returned (same offset).  The owner must keep
 *       the block allocated until every importer has released it.
 */
#define DSDPA_PEER_HANDLE_BYTES 64
int dsdpa_peer_export(const void* ptr, int device, unsigned char handle[DSDPA_PEER_HANDLE_BYTES], size_t* offset);
int dsdpa_peer_import(const unsigned char handle[DSDPA_PEER_HANDLE_BYTES], size_t offset, int device, void** ptr);
int dsdpa_peer_release(void* ptr, size_t offset, int device);

/*
 * Backward without caller-provided scratch.  (No counterpart in the reference: its backward
 * allocates its accumulators with torch on every call, ops/triton.py:427-430, which is
 * exactly what the callers of this entry point are not allowed to do.)
 *
 * For callers that cannot allocate device memory at the point where the backward runs --
 * a serving loop with a frozen memory budget, a plugin inside a host that owns the device
 * heap, a callback running under the allocator's lock -- the scratch dsdpa_backward asks
 * its caller for is taken from a fixed array that is part of the library image:
 * DSDPA_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, from
 * load until process exit.  The call allocates and frees nothing (no cudaMalloc/cudaFree,
 * no allocating library routine); inputs and outputs are still the caller's.
 *
 *   - Same results, arguments and flags as dsdpa_backward with dcoords == NULL.
 *   - A problem whose dsdpa_backward_workspace_bytes exceeds DSDPA_STATIC_SCRATCH_BYTES is
 *     refused with DSDPA_ERR_TOO_LARGE before any work is enqueued.
 *   - The first call on a device looks up the array's device address.  The array belongs to the
 *     library's device image; where the CUDA runtime loads modules lazily, the driver may place
 *     that image -- and with it reserve the DSDPA_STATIC_SCRATCH_BYTES -- only at this first
 *     call, which can therefore fail with an out-of-memory DSDPA_ERR_CUDA on a full device.
 *     Make that first call once per device during initialisation, outside any stream capture;
 *     later calls touch no allocator of any kind.
 *   - All calls on a device share the one array, which keeps the previous call's contents;
 *     what has to start at zero is cleared on `stream` by every call.  Calls whose GPU work
 *     overlaps (other streams, other host threads) race on it: keep them on one stream.
 */
#define DSDPA_STATIC_SCRATCH_BYTES (64u << 20)
int dsdpa_backward_static_scratch(const dsdpa_problem* p,
                                  const void* q, const void* k, const void* v, const float* coords,
                                  const void* out, const float* lse, const void* dout,
                                  void* dq, void* dk, void* dv, int device, void* stream);

/* Human-readable name of a dsdpa_status. */
const char* dsdpa_status_string(int status);

/* DSDPA_VERSION of the loaded library. */
int dsdpa_version(void);

/* Kernels of this library launched by this process so far (memsets are not counted). */
unsigned long long dsdpa_kernel_launches(void);

/* cudaError_t value of the last failed CUDA call of this thread's last DSDPA_ERR_CUDA. */
int dsdpa_last_cuda_error(void);

/*
 * Synchronises `device` and returns DSDPA_ERR_DEVICE_TIMEOUT if any kernel of this
 * library recorded that a bounded wait ran out since the last call (clearing the
 * record), DSDPA_ERR_DEVICE_BOUNDS if a kernel of the checked build found an index out of
 * range, DSDPA_OK otherwise.  A kernel that gave up returns without writing its results, and
 * nothing else reports that: callers who need to know poll this function.
 */
int dsdpa_device_error(int device);

/*
 * Self-test of the bounded wait every kernel's mbarrier waits go through (no counterpart in
 * the reference, which has no device-side waits): enqueues one warp that waits on a barrier
 * nobody completes, gives up after `polls` polls (1 .. 2^20), records the timeout and returns.
 * dsdpa_device_error(device) then answers DSDPA_ERR_DEVICE_TIMEOUT once.  Nothing hangs or
 * faults; the context stays usable.
 */
int dsdpa_selftest_bounded_wait(unsigned polls, int device, void* stream);

/* 1 if this library was built with -DDSDPA_BOUNDS_CHECK (the checked debug build), else 0. */
int dsdpa_build_is_checked(void);

/*
 * How the library would run this problem: fills `text` (up to `cap` bytes, NUL
 * terminated) with a one-line description (paths, tile sizes, shared memory).
 */
int dsdpa_describe_plan(const dsdpa_problem* p, char* text, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* DSDPA_H_ */
