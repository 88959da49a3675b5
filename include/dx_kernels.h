/*
 * dx_kernels.h — C ABI of the B200 (sm_100a) tensor-function kernels.
 *
 * This is the seam where the deepx executor's `launch_*<T>` host wrappers sit
 * in the reference (the .cuh files of executor/op-cuda/src/deepx/tensorfunc/).  Every entry
 * point takes plain device pointers, sizes and a CUDA stream handle; nothing is
 * allocated inside a call, nothing throws.  Return value: DX_OK (0) or a
 * negative DX_E_* code; dx_last_error() gives the message of the last failure
 * on the calling thread.
 *
 * All tensors are row-major contiguous (deepx::Shape semantics,
 * executor/deepxcore/src/deepx/shape.cpp:21-32) with 64-bit extents.
 * Element counts are int64_t; rank is at most DX_MAX_DIMS.
 * `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Output buffers may alias an input buffer only where a function says so.
 */
#ifndef DX_KERNELS_H
#define DX_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DX_MAX_DIMS 12 /* executor/op-cuda/src/deepx/tensorfunc/tensor_cuda.cuh:38 */

/* dtype codes: the tensor precisions of executor/deepxcore/src/deepx/dtype.hpp:120-146
 * that op-cuda instantiates kernels for. */
typedef enum {
    DX_F64 = 0,
    DX_F32 = 1,
    DX_F16 = 2,
    DX_BF16 = 3,
    DX_I64 = 4,
    DX_I32 = 5,
    DX_I16 = 6,
    DX_I8 = 7,
    DX_BOOL = 8,
    DX_DTYPE_COUNT = 9
} dx_dtype;

typedef enum {
    DX_OK = 0,
    DX_E_DTYPE = -1,     /* dtype not supported by this op */
    DX_E_SHAPE = -2,     /* shape / rank / axis invalid */
    DX_E_ARG = -3,       /* null pointer, bad op code, bad count */
    DX_E_CUDA = -4,      /* CUDA runtime / driver error; message has the string */
    DX_E_WORKSPACE = -5, /* workspace missing or too small */
    DX_E_ALIAS = -6,     /* output overlaps an input where that is not defined */
    DX_E_UNSUPPORTED = -7
} dx_status;

const char *dx_last_error(void);
/* Size in bytes of one element of `dtype`, 0 if unknown. */
int dx_dtype_size(int dtype);
/* Number of SMs of the current device (cached per device). */
int dx_sm_count(void);
/* Kernels this library has launched in this process so far (all threads, all devices). */
unsigned long long dx_launch_count(void);

/* ---- elementwise: tensor ∘ tensor ---------------------------------------
 * Replaces launch_add/sub/mul/div/max/min/pow
 * (executor/op-cuda/src/deepx/tensorfunc/elementwise_miaobyte_basic.cuh:23-77,
 *  elementwise_miaobyte_compare.cuh:13-40, elementwise_miaobyte_sqrt.cuh:18-24).
 * c may alias a and/or b exactly (same base pointer). */
typedef enum {
    DX_ADD = 0,
    DX_SUB = 1,
    DX_MUL = 2,
    DX_DIV = 3,
    DX_MAX = 4,
    DX_MIN = 5,
    DX_POW = 6, /* f64, f32 only */
    DX_BINARY_COUNT = 7
} dx_binary_op;
int dx_ew_binary(int op, int dtype, const void *a, const void *b, void *c, int64_t n, void *stream);

/* ---- elementwise: tensor ∘ scalar ---------------------------------------
 * Replaces launch_addscalar/subscalar/rsubscalar/mulscalar/divscalar/rdivscalar,
 * maxscalar/minscalar, powscalar/rpowscalar (same files as above).
 * The scalar is `fscalar` for floating dtypes (narrowed to the tensor dtype) and
 * `iscalar` for integer dtypes.  c may alias a exactly. */
typedef enum {
    DX_ADDS = 0,
    DX_SUBS = 1,  /* a - s */
    DX_RSUBS = 2, /* s - a */
    DX_MULS = 3,
    DX_DIVS = 4,  /* a / s */
    DX_RDIVS = 5, /* s / a */
    DX_MAXS = 6,
    DX_MINS = 7,
    DX_POWS = 8,  /* pow(a, s)  f64, f32 only */
    DX_RPOWS = 9, /* pow(s, a)  f64, f32 only */
    DX_SCALAR_COUNT = 10
} dx_scalar_op;
int dx_ew_scalar(int op, int dtype, const void *a, double fscalar, int64_t iscalar, void *c, int64_t n,
                 void *stream);

/* ---- elementwise: unary --------------------------------------------------
 * Replaces launch_sqrt/log/exp (elementwise_miaobyte_sqrt.cuh:10-56),
 * launch_sin/cos/tan (elementwise_miaobyte_sin.cuh) and launch_invert
 * (elementwise_miaobyte_basic.cuh:95-99).  c may alias a exactly. */
typedef enum {
    DX_SQRT = 0,
    DX_LOG = 1,
    DX_EXP = 2,
    DX_SIN = 3,
    DX_COS = 4,
    DX_TAN = 5,
    DX_INVERT = 6, /* ~a for i64/i32/i16/i8, !a for bool */
    DX_UNARY_COUNT = 7
} dx_unary_op;
int dx_ew_unary(int op, int dtype, const void *a, void *c, int64_t n, void *stream);

/* ---- elementwise: compare → bool mask -------------------------------------
 * Replaces launch_equal/notequal/less/greater and their *scalar forms
 * (elementwise_miaobyte_compare.cuh:43-117).  mask is one byte per element
 * (0/1).  epsilon is used by EQ/NE only: epsilon==0 → exact compare, otherwise
 * EQ = |a-b| <= epsilon and NE = |a-b| > epsilon, the op-ompsimd rule
 * (executor/op-ompsimd/src/deepx/tensorfunc/elementwise_miaobyte.hpp:778-845). */
typedef enum { DX_EQ = 0, DX_NE = 1, DX_LT = 2, DX_GT = 3, DX_COMPARE_COUNT = 4 } dx_compare_op;
int dx_ew_compare(int op, int dtype, const void *a, const void *b, float epsilon, void *mask, int64_t n,
                  void *stream);
int dx_ew_compare_scalar(int op, int dtype, const void *a, double fscalar, int64_t iscalar, float epsilon,
                         void *mask, int64_t n, void *stream);

/* ---- switch (where) ------------------------------------------------------
 * Replaces launch_switch (elementwise_miaobyte_compare.cuh:112-117):
 * c[i] = tensors[cases[i]][i].  cases_dtype is DX_BOOL (ntensors must be 2:
 * false→tensors[0], true→tensors[1]) or DX_I32.  `tensors` is a HOST array of
 * ntensors (≤ DX_SWITCH_MAX) device pointers; it is copied into the kernel
 * parameters, so no device-side pointer table is needed. */
#define DX_SWITCH_MAX 16
int dx_switch(int dtype, const void *const *tensors, int ntensors, int cases_dtype, const void *cases, void *c,
              int64_t n, void *stream);

/* ---- todtype -------------------------------------------------------------
 * Replaces launch_todtype (elementwise_miaobyte_basic.cuh:13-14): static_cast
 * semantics between any two of f64,f32,f16,bf16,i64,i32,i16,i8 (+bool).
 * Same dtype = plain copy. */
int dx_cast(int src_dtype, const void *a, int dst_dtype, void *c, int64_t n, void *stream);

/* ---- constant fill -------------------------------------------------------
 * Replaces launch_constant (init_miaobyte.cuh:11). */
int dx_fill(int dtype, void *c, double fscalar, int64_t iscalar, int64_t n, void *stream);

/* ---- initialisers ----------------------------------------------------------
 * Replace launch_arange/uniform/normal/dropout (init_miaobyte.cuh:19-47).
 * arange: out[i] = T(float(start) + float(step) * float(i)), the reference's fp32 form.
 * uniform [low, high), normal(mean, stddev), dropout (zero with probability p, in place):
 * element i depends on (seed, i) only. */
int dx_arange(int dtype, void *out, double start, double step, int64_t n, void *stream);
int dx_uniform(int dtype, void *out, double low, double high, uint64_t seed, int64_t n, void *stream);
int dx_normal(int dtype, void *out, double mean, double stddev, uint64_t seed, int64_t n, void *stream);
int dx_dropout(int dtype, void *inout, double p, uint64_t seed, int64_t n, void *stream);

/* ---- reduce ----------------------------------------------------------------
 * Replaces launch_sum/prod/reducemax/reducemin (reduce_miaobyte.cuh:16-56).
 * Reduces `a` (row-major `shape[ndim]`) over the axes in `dims[ndims]`
 * (already normalised: 0 ≤ d < ndim, sorted, unique — what checkedDims,
 * executor/deepxcore/src/deepx/shape_reduce.cpp:11-45, produces) into `out`
 * (row-major over the kept axes; keepdims only changes the shape metadata, not
 * the element order).  Deterministic: no atomics, fixed combine order.
 * Some shapes need device scratch for the cross-block pass: query it with
 * dx_reduce_workspace_bytes() and pass a buffer at least that large (256-byte
 * aligned); 0 means none is needed.  out must not alias a. */
typedef enum { DX_SUM = 0, DX_PROD = 1, DX_RMAX = 2, DX_RMIN = 3, DX_REDUCE_COUNT = 4 } dx_reduce_op;
size_t dx_reduce_workspace_bytes(int op, int dtype, const int64_t *shape, int ndim, const int32_t *dims,
                                 int ndims);
int dx_reduce(int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims,
              void *out, void *workspace, size_t workspace_bytes, void *stream);

/* Reduce for callers that cannot allocate device memory.  No counterpart in the reference.
 * Same arguments and results as dx_reduce, minus the workspace: the cross-block scratch is a
 * 1 MiB array built into the library image (present on every GPU that loads the library, for
 * the life of the process).  Meant for hosts that have given their whole memory budget to a
 * pre-sized pool, that run inside another allocator's callback, or that ban cudaMalloc after
 * start-up because it stalls the device.  The call itself allocates and frees no device memory.
 *  - A shape whose scratch need exceeds 1 MiB is refused with DX_E_WORKSPACE (the message gives
 *    both sizes); use dx_reduce with your own workspace for those.
 *  - The first call on each device looks up the array's device address (that device must be
 *    current); make that first call before starting any stream capture.
 *  - All calls on a device share the one array: calls that can overlap on the GPU (different
 *    streams or threads) race on it.  Issue them on one stream.  The array is not cleared
 *    between calls and does not need to be. */
int dx_reduce_noalloc(int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims,
                      int ndims, void *out, void *stream);

/* ---- cross-GPU combine (no reference counterpart: the reference is single-GPU) ----
 * One process per GPU.  A reduction over the axis a tensor is sharded along leaves one partial
 * per rank; dx_comm_allreduce combines them IN PLACE with one kernel per rank that stores its
 * partial into every peer's mailbox over NVLink peer memory and combines the W partials in rank
 * order (identical bits on every rank).  A buffer larger than dx_comm_max_bytes() (one mailbox slot)
 * goes in several rounds of the same kernel.  Set-up: every rank calls dx_comm_create, exchanges the 64-byte handles
 * of dx_comm_handle by any host channel, and gives all of them (world x 64 bytes, rank order) to
 * dx_comm_connect.  All ranks must issue the same sequence of dx_comm_allreduce calls.
 * Waits on a peer are bounded (2 s unless dx_comm_set_timeout_ms): when one expires the kernel
 * leaves the local buffer untouched and returns; dx_comm_status (synchronises the stream) then
 * reports DX_E_CUDA with the peer it gave up on, and the communicator should be discarded. */
typedef struct dx_comm dx_comm;
size_t dx_comm_max_bytes(void);
dx_comm *dx_comm_create(int rank, int world, int device);
int dx_comm_handle(dx_comm *c, unsigned char out[64]);
int dx_comm_connect(dx_comm *c, const unsigned char *handles);
int dx_comm_set_timeout_ms(dx_comm *c, int ms);
int dx_comm_allreduce(dx_comm *c, int op, int dtype, void *buf, int64_t n, void *stream);
int dx_comm_status(dx_comm *c, void *stream);
/* What the rendezvous has cost this rank since the counters were last reset: the number of flag waits its CTAs did
 * and the time they took (per CTA the longest of its threads, summed; SM cycles at the device's nominal clock,
 * given in microseconds).  Synchronises the stream.  A wait that finds its flags already set counts a few hundred
 * nanoseconds: the round trip of the acquire loads. */
int dx_comm_wait_stats(dx_comm *c, double *microseconds, long long *waits, int reset, void *stream);
void dx_comm_destroy(dx_comm *c);
int dx_comm_rank(dx_comm *c);
int dx_comm_world(dx_comm *c);
/* The all-reduce in two halves.  _begin stores this rank's buffer (at most dx_comm_max_bytes()) into the
 * peers' mailboxes and raises its flags, without waiting for anybody; _finish waits (bounded) for the
 * peers' flags and combines in place.  Kernels launched on the stream between the two run while the
 * slower ranks catch up, so the per-step skew between ranks is hidden instead of waited out.  One
 * exchange can be outstanding per communicator: a second _begin, dx_comm_allreduce,
 * dx_comm_allgather_rows or dx_reduce_allreduce* first finishes the one before (on ITS stream argument).
 * The buffer must not be read or written between _begin and _finish.  dx_comm_pending returns 1 and the
 * buffer while an exchange is outstanding. */
int dx_comm_allreduce_begin(dx_comm *c, int op, int dtype, void *buf, int64_t n, void *stream);
int dx_comm_allreduce_finish(dx_comm *c, void *stream);
int dx_comm_pending(dx_comm *c, void **buf);
/* Contiguous split of `global_rows` leading-axis indices over `world` ranks (the first
 * global_rows % world ranks get one row more): where rank's block starts and how many rows it has. */
void dx_shard_rows(int64_t global_rows, int rank, int world, int64_t *row0, int64_t *rows);
/* All-gather of row blocks, in place: every rank holds the whole [global_rows x row_bytes] buffer and has
 * filled its own block (dx_shard_rows); afterwards every rank holds every block.  Peer stores and the
 * same bounded flag waits as the all-reduce; blocks larger than a mailbox slot go in rounds. */
int dx_comm_allgather_rows(dx_comm *c, void *buf, int64_t global_rows, int64_t row_bytes, void *stream);
/* dx_reduce on this rank's shard followed by the combine over the ranks, result on every rank.
 * Where the local reduction ends in a one-CTA finish step (few outputs — the global sum of a sharded
 * tensor is one) that CTA also performs the exchange, so a single launch is the tail of the
 * reduction and the all-reduce; otherwise the exchange kernel follows on the same stream.  The
 * output must fit dx_comm_max_bytes(); workspace as for dx_reduce. */
int dx_reduce_allreduce(dx_comm *c, int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims,
                        void *out, void *workspace, size_t workspace_bytes, void *stream);
/* The same, stopping after this rank's result has been published to the peers (by the reduction's own
 * finish kernel where it has one): dx_comm_allreduce_finish completes it. */
int dx_reduce_allreduce_begin(dx_comm *c, int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims,
                              void *out, void *workspace, size_t workspace_bytes, void *stream);
/* The same protocol with every rank on ONE GPU (all mailboxes local, all ranks' CTAs in one
 * launch, which is the only safe way to run kernels that wait on each other on one device):
 * bufs[r] is rank r's buffer.  Ranks >= active_ranks are left out, so the others' waits expire
 * and dx_comm_status reports it — the failure path without a misbehaving process. */
dx_comm *dx_comm_emulate(int world, int device);
int dx_comm_emulated_allreduce(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream);
/* The two halves of the exchange as separate launches, and the row-block all-gather, on emulated ranks. */
int dx_comm_emulated_publish(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream);
int dx_comm_emulated_combine(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream);
int dx_comm_emulated_allgather_rows(dx_comm *c, void *const *bufs, int64_t global_rows, int64_t row_bytes, void *stream);

/* ---- fused row chains --------------------------------------------------------
 * The reference has no single function for these: its front end builds RMSNorm
 * (front/py/deepx/nn/modules/norm/t5layernorm.py:19-23) and softmax
 * (front/py/deepx/nn/functional/normalization.py:4-18) out of single ops, one
 * kernel launch and one pass over HBM each.  These two calls run such a chain
 * over contiguous rows in one pass (the row stays in registers).  Each step uses
 * the arithmetic of the single op it stands for, rounding to `dtype` included,
 * so the result differs from the op-by-op chain only by the order of the
 * additions inside the row sum.  Float dtypes only.  `out` may alias `x`.
 *
 * dx_rmsnorm: out[r,i] = weight[i] * (x[r,i] * (1 / sqrt(sum_i(x[r,i]^2) / divisor + eps)))
 *             — powscalar(x,2)|mul(x,x), sum(last,keepdims), divscalar(divisor),
 *             addscalar(eps), sqrt, rdivscalar(1), broadcastTo, mul, [broadcastTo(weight), mul].
 *             `weight` (cols elements) may be NULL: the last multiply is then left out.
 * dx_softmax: m = max_i x[r,i]; e_i = exp(x[r,i] - m); out[r,i] = e_i / sum_i e_i
 *             — reducemax(last,keepdims), broadcastTo, sub, exp, sum(last,keepdims), broadcastTo, div. */
int dx_rmsnorm(int dtype, const void *x, const void *weight, void *out, int64_t rows, int64_t cols, double divisor,
               double eps, void *stream);
int dx_softmax(int dtype, const void *x, void *out, int64_t rows, int64_t cols, void *stream);

/* ---- changeshape -----------------------------------------------------------
 * Replace launch_transpose/concat/broadcastTo/indexselect/repeat
 * (changeshape_miaobyte.cuh:16-88).  Pure data movement, bit-exact for every
 * dtype (selected by element size).  Outputs must not alias inputs. */

/* out.shape[i] = shape[perm[i]]  (transposeShape, shape_changeshape.cpp:17-29) */
int dx_transpose(int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *perm, void *out,
                 void *stream);

/* inputs: HOST array of ninputs device pointers; axis_len[i] = extent of input i
 * on `axis`; out_shape is the result shape (its extent on `axis` = Σ axis_len). */
int dx_concat(int dtype, const void *const *inputs, const int64_t *axis_len, int ninputs,
              const int64_t *out_shape, int ndim, int axis, void *out, void *stream);

/* numpy-style right-aligned broadcast of a (a_shape[a_ndim]) to out_shape[out_ndim]
 * (broadcastMap, shape_changeshape.cpp:81-105). */
int dx_broadcast_to(int dtype, const void *a, const int64_t *a_shape, int a_ndim, const int64_t *out_shape,
                    int out_ndim, void *out, void *stream);

/* Gather along `axis` with an index TENSOR (any rank): out.shape =
 * a.shape[:axis] + idx.shape + a.shape[axis+1:]  (indexselectShape,
 * shape_changeshape.cpp:122-141).  idx_dtype is DX_I32 or DX_I64.  An index
 * outside [0, a.shape[axis]) writes zeros for that slice and raises bit 0 of
 * *oob_flag (device int32, may be NULL). */
int dx_indexselect(int dtype, const void *a, const int64_t *a_shape, int a_ndim, int idx_dtype, const void *idx,
                   const int64_t *idx_shape, int idx_ndim, int axis, void *out, int32_t *oob_flag,
                   void *stream);

/* out[i] = a[i / repeats] per axis (repeatShape, shape_changeshape.cpp:144-156). */
int dx_repeat(int dtype, const void *a, const int64_t *a_shape, int ndim, const int64_t *repeats, void *out,
              void *stream);

/* ---- matmul ----------------------------------------------------------------
 * Replaces matmulDispatcher<cublas,T>::matmul
 * (executor/op-cuda/src/deepx/tensorfunc/matmul_cublas.hpp:16-145): batched
 * row-major C[b,M,N] = A[b,M,K] · B[b,K,N], all three the same dtype.
 * DX_BF16 / DX_F16: tcgen05 tensor-core kernel, fp32 accumulation in TMEM,
 * one rounding to the output dtype.  DX_F32 / DX_F64: SIMT FMA kernel with
 * accumulation in the tensor dtype. */
int dx_matmul(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K,
              void *stream);
/* The same with scratch memory from the caller.  A matrix with a few rows of 256 x 256 tiles (M of a few hundred)
 * gives too few tiles for the SMs; with a workspace the K range of each tile is split over several CTA pairs
 * (a cooperative launch: all of them resident), whose fp32 partials meet in the workspace; every pair finishes
 * its share of the tile's columns, adding in a fixed order (same bits every run, no atomics on data).
 * dx_matmul_workspace_bytes says how much that takes for a shape on the current device (0: the shape does not
 * use a workspace); with less (or NULL) the call does what dx_matmul does.  A workspace serves one stream at a
 * time; calls on different streams, each with its own workspace, may overlap (up to 8 streams per device take
 * this path, further ones do what dx_matmul does). */
size_t dx_matmul_workspace_bytes(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K);
int dx_matmul_ws(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                 void *workspace, size_t workspace_bytes, void *stream);
/* Every wait inside the tensor-core kernel is bounded; if one expires the kernel records
 * which and returns.  This reads (and clears) that record: DX_OK, or DX_E_CUDA with the
 * stage in the message.  Synchronises `stream`.  Stands where the reference checks
 * cudaGetLastError after a launch (executor/op-cuda/src/deepx/tensorfunc/cuda.hpp:73-78). */
int dx_matmul_status(void *stream);

/* ---- device memory pool ------------------------------------------------------
 * Replaces the per-tensor cudaMalloc/cudaFree of
 * executor/op-cuda/src/deepx/tensorfunc/tensorlife_miaobyte.hpp:16-40 and the
 * empty MemoryPool stub (new_mempool.hpp:6-37): one caching pool per device,
 * 256-byte aligned blocks, size-class free lists, blocks returned to the pool
 * are reusable by later work on the same stream order. */
typedef struct dx_pool dx_pool;
dx_pool *dx_pool_create(int device, size_t max_bytes /* 0 = unlimited */);
void dx_pool_destroy(dx_pool *pool);
void *dx_pool_alloc(dx_pool *pool, size_t bytes);
int dx_pool_free(dx_pool *pool, void *ptr);
/* stats[0]=bytes in use, [1]=bytes reserved from the driver, [2]=high-water in use, [3]=#cudaMalloc calls */
void dx_pool_stats(const dx_pool *pool, size_t stats[4]);
/* Return all cached (free) blocks to the driver. */
void dx_pool_trim(dx_pool *pool);

#ifdef __cplusplus
}
#endif
#endif /* DX_KERNELS_H */
