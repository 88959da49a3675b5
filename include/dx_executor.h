/*
 * dx_executor.h — C ABI of the deepxIR executor (libdeepx_exec.so).
 *
 * One handle = what one reference executor process holds: the tensor store (`Mem`,
 * executor/deepxcore/src/deepx/mem/mem.hpp), the op registry filled by register_all
 * (executor/op-cuda/src/client/tfs.cpp:636-646) and a device pool + stream.  dx_exec_run takes
 * one deepxIR text line and produces the reply line the reference's main loop would send over
 * UDP (executor/op-cuda/src/client/main.cpp:47-102, reply format tf.hpp:198-213); the
 * `deepx-op-b200` binary is exactly this behind a UDP socket.  The upload/download calls are the
 * in-process stand-in for the on-disk tensor exchange (save/load IR ops work too).
 * All functions return 0 on success and a negative value on failure unless stated otherwise.
 *
 * Threads: an executor handle is for ONE thread at a time, as the reference's executor has one
 * worker thread (main.cpp:25,74,93).  dx_exec_run serialises itself, but upload / download / bind /
 * tensor_info / compile touch the tensor store and the compute stream without a lock, and a program
 * being compiled keeps a stream capture open across several internal runs: do not call into the
 * same handle from a second thread meanwhile.  Different handles are independent.
 */
#ifndef DX_EXECUTOR_H
#define DX_EXECUTOR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dx_exec dx_exec;

/* pool_limit_bytes = 0: no limit.  NULL on failure (dx_exec_last_error has the reason). */
dx_exec *dx_exec_create(int device, size_t pool_limit_bytes);
void dx_exec_destroy(dx_exec *e);
const char *dx_exec_last_error(void);

/* Runs one IR line.  Writes the NUL-terminated reply ("<id> ok// recv_at=… start_at=… finish_at=…"
 * or "<id> error// … <message>") into reply[cap].  Returns 0 when the op succeeded, 1 when the
 * reply is an error reply, -1 when reply does not fit. */
int dx_exec_run(dx_exec *e, const char *ir_line, char *reply, size_t cap);

/* Runs a program: several IR lines in one text, one per line (what one UDP datagram may carry,
 * executor/deepxcore/src/client/udpserver.cpp:49-58).  The replies, one per non-empty line and in
 * order, are written into replies[cap] separated by '\n'.  Before running, the fusion pass looks
 * for the op chains the front end emits for RMSNorm
 * (front/py/deepx/nn/modules/norm/t5layernorm.py:19-23) and softmax
 * (front/py/deepx/nn/functional/normalization.py:4-18); a chain whose intermediate tensors are
 * created and deleted inside the program and used by nothing else runs as ONE kernel
 * (dx_rmsnorm / dx_softmax), and the lines it absorbed are answered "ok" without running.  The
 * reference has no such pass (one launch per line).  Returns the number of error replies, or -1
 * when the replies do not fit. */
int dx_exec_run_program(dx_exec *e, const char *program, char *replies, size_t cap);
/* Fusion on (default) / off for dx_exec_run_program. */
void dx_exec_set_fusion(dx_exec *e, int on);
/* [0] programs seen, [1] RMSNorm chains rewritten, [2] softmax chains rewritten, [3] IR lines absorbed. */
void dx_exec_fusion_stats(dx_exec *e, uint64_t stats[4]);

/* A program whose kernels are captured once into a CUDA graph and replayed with one launch call:
 * for sequences of small ops the host cost per IR line is what limits throughput, and a replay
 * has none of it (the reference pays a UDP round trip per line).  The program may only compute:
 * tensor lifetime, io and arg ops, timed lines, and ops that would need a temporary are refused;
 * op chains the fusion pass absorbs (with their temporaries) are fine.  dx_exec_compile runs the
 * program once — those results stand — and captures a second pass; NULL on failure
 * (dx_exec_last_error).  dx_program_run checks that every tensor the program names still has the
 * same storage, dtype and shape, then launches the graph on the executor's stream (asynchronous);
 * 0 ok, 1 = stale or failed (dx_exec_last_error), and the program must be compiled again.
 * info: [0] IR lines, [1] ops captured after fusion, [2] graph nodes, [3] fused chains.
 * Free programs before destroying their executor. */
typedef struct dx_program dx_program;
dx_program *dx_exec_compile(dx_exec *e, const char *program);
int dx_program_run(dx_program *p);
void dx_program_info(dx_program *p, size_t info[4]);
void dx_program_free(dx_program *p);

/* Registers device memory the executor does not own (a heap tensor mapped with dx_heap_open, a
 * buffer of the embedding application) as tensor `name`, so IR ops can read and write it.  The
 * executor never frees it; deltensor only forgets the name.  The memory must stay valid, on the
 * executor's device, while the name is registered.  Fails if the name exists. */
int dx_exec_bind_tensor(dx_exec *e, const char *name, int dtype, const int64_t *shape, int ndim, void *device_ptr);

/* ---- one executor per GPU, several GPUs (no reference counterpart: the reference has one Mem and one device,
 * executor/op-cuda/src/client/main.cpp:22-105, executor/heapmem-cuda/README.md:19,29) ----
 * Makes this executor rank `rank` of `world`: one process per GPU, every rank is given the SAME IR lines, `comm`
 * is a connected dx_comm (dx_kernels.h) for this rank and must outlive the executor.  From then on newtensor
 * partitions a tensor by rows (contiguous blocks of its leading axis, dx_shard_rows) when it holds at least
 * `min_bytes` and has at least `world` rows; smaller tensors are replicated on every rank.  Ops that work row
 * by row run on the local rows without communication; a reduction that removes axis 0 combines the ranks'
 * partials over NVLink peer memory (its wait for the peers is left until the result is next needed, so the ops
 * in between hide the skew between ranks); ops with no row-wise form refuse partitioned operands with an
 * error reply.  save writes, and load / loadtensordata read, the very files a single GPU would (each rank its
 * rows).  Upload, download, tensor_info and tensor_ptr see the LOCAL rows of a partitioned tensor. */
typedef struct dx_comm dx_comm;
int dx_exec_set_shard(dx_exec *e, int rank, int world, size_t min_bytes, dx_comm *comm);
/* Where a tensor's rows sit: first row and number of rows held by this rank, and the global row count.
 * Returns 1 if the tensor is partitioned, 0 if it is whole (replicated), -1 if there is no such tensor. */
int dx_exec_tensor_shard(dx_exec *e, const char *name, int64_t *row0, int64_t *rows, int64_t *global_rows);
/* The partition decisions alone, without a GPU: for every line of `program` what a rank of `world` would do with
 * it — "newtensor <name>: partitioned <rows> rows" / "whole", "rows", "rows+allgather", "whole",
 * "allreduce(deferred)", "allreduce(rounds)", "allreduce(rounds)+keep-own-rows", "rows-if-aligned" (changeshape,
 * matmul and fused ops: by rows where the operands' rows line up, refused otherwise) or "refuse: <why>" — one per
 * line, '\n'-separated.  Returns the number of lines, -1 on a parse error (dx_exec_last_error). */
int dx_ir_shard_plan(const char *program, int world, size_t min_bytes, char *out, size_t cap);

/* Tensor metadata: dtype is a dx_dtype code; shape receives up to cap extents (the local rows of a
 * partitioned tensor); returns the rank, or -1 if there is no such tensor. */
int dx_exec_tensor_info(dx_exec *e, const char *name, int *dtype, int64_t *shape, int cap);
/* Device pointer of a tensor's storage (NULL if absent). */
void *dx_exec_tensor_ptr(dx_exec *e, const char *name);
/* Copies host bytes into / out of an existing tensor (exactly its size in bytes). Synchronous. */
int dx_exec_upload(dx_exec *e, const char *name, const void *host, size_t bytes);
int dx_exec_download(dx_exec *e, const char *name, void *host, size_t bytes);
/* Upload without waiting: the copy runs on a stream of its own, ordered behind everything submitted so far; the
 * first op (or download) that names the tensor afterwards waits for it on the device, other ops do not.  `host`
 * must stay valid, and should be page-locked for the copy to overlap with compute, until dx_exec_sync or a
 * download of a result that depends on it. */
int dx_exec_upload_async(dx_exec *e, const char *name, const void *host, size_t bytes);
/* Waits for everything submitted so far. */
int dx_exec_sync(dx_exec *e);
/* The executor's CUDA stream (cudaStream_t as void*). */
void *dx_exec_stream(dx_exec *e);
/* Markdown op table (TfFactory::print_markdown, tffactory.cpp:85-119); returns bytes needed. */
size_t dx_exec_op_table(dx_exec *e, char *out, size_t cap);
/* Pool statistics as dx_pool_stats, plus [4] = ops run. */
void dx_exec_stats(dx_exec *e, size_t stats[5]);

/* Parser / registry probes that need no GPU (used by the differential tests):
 * canonical one-line rendering of what the parser understood:
 * "<name>|<arg dtype>:<arg text>,…|<ret dtype>:<ret text>,…|author=<a> id=<n> repeat=<n>", or "!<error>". */
int dx_ir_parse(const char *ir_line, char *out, size_t cap);
int dx_ir_dtype_roundtrip(const char *text, char *out, size_t cap);
/* The integer vector argument `arg_index` of an IR line (extents, repeats) as the executor reads it:
 * 64-bit, plain integer text exactly, other numeric text through std::stof as the reference's to<int>
 * does (executor/deepxcore/src/deepx/dtype.hpp:15-25).  Returns the count, or -1 (dx_exec_last_error). */
int dx_ir_vector_i64(const char *ir_line, int arg_index, int64_t *out, int cap);
/* print's format argument (executor/deepxcore/src/stdutil/print.hpp:13-57 hands it to printf unchecked):
 * accepted only with exactly one numeric conversion that fits the tensor's dtype; `out` gets the format
 * actually used (length modifier normalised).  0 = accepted, 1 = refused (dx_exec_last_error says why). */
int dx_ir_check_print_format(const char *format, int dtype, char *out, size_t cap);
/* The fusion pass alone, no GPU needed.  `existing` lists tensors that exist before the program,
 * one per line as "<name> <dtype name> <d0> <d1> …" (may be NULL or empty).  Writes one line per
 * program line: "run", "absorbed <group>" or "fused <group> <the op that runs instead>".
 * Returns the number of fused groups, or -1 (parse error, or the text does not fit). */
int dx_ir_plan_fusion(const char *program, const char *existing, char *out, size_t cap);
/* A registry without an executor: add signature lines, ask which registration a call resolves to. */
void *dx_registry_new(int with_builtin_ops);
void dx_registry_free(void *r);
int dx_registry_add(void *r, const char *signature_ir);
int dx_registry_get(void *r, const char *call_ir); /* index in registration order, -1 = no match */
int dx_registry_size(void *r);

#ifdef __cplusplus
}
#endif
#endif
