/* b200mk.h - C ABI of the B200 persistent decode megakernel.
 *
 * Plain C, no torch or C++ types: every pointer is a raw device or host
 * address, every size an integer.  The entry points are what a binding of the
 * reference's MPK operator API needs for the decode path; each one names the
 * reference interface it stands in for (paths relative to the reference tree).
 *
 * All functions return 0 (or a non-negative id) on success and a negative
 * MK_E_* code on failure; mk_last_error() gives the message.  Nothing here
 * calls exit().  A handle is not thread-safe; use one handle per GPU.
 */
#ifndef B200MK_H
#define B200MK_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mk_handle mk_handle;

enum { MK_BF16 = 0, MK_F32 = 1, MK_I32 = 2, MK_I64 = 3, MK_U64 = 4, MK_F16 = 5 };
enum { MK_MODE_OFFLINE = 0, MK_MODE_ONEPASS = 1 };
enum { MK_NUMERICS_MPK = 0, MK_NUMERICS_TORCH = 1 };
enum { MK_CAT_CUDA = 0, MK_CAT_SYMMETRIC = 1 };
enum {
  MK_E_INVALID = -1,   /* bad argument, shape or dtype */
  MK_E_STATE = -2,     /* call out of order (e.g. launch before compile) */
  MK_E_CUDA = -3,      /* a CUDA runtime/driver call failed */
  MK_E_UNSUPPORTED = -4,
  MK_E_DEVICE = -5,    /* the kernel reported a timeout or bad data; see mk_last_error */
  MK_E_NOMEM = -6,
  MK_E_TOO_LARGE = -7  /* a size beyond a fixed built-in limit */
};

/* Constructor arguments of PersistentKernel
 * (python/mirage/mpk/persistent_kernel.py:368-387). */
typedef struct mk_config {
  int32_t mode;                     /* MK_MODE_* ("offline" / "online_notoken") */
  int32_t world_size;
  int32_t rank;                     /* mpi_rank */
  int32_t num_workers;              /* hint; 0 = one CTA per SM */
  int32_t max_seq_length;
  int32_t max_num_batched_requests;
  int32_t max_num_batched_tokens;
  int32_t max_num_pages;
  int32_t page_size;
  int32_t numerics;                 /* MK_NUMERICS_* */
  int64_t eos_token_id;
  int32_t fuse;                     /* 1 = fuse norm/SiLU/argmax into the linear tasks */
  int32_t max_iterations;           /* 0 = run until every request has finished */
  int64_t timeout_ms;               /* bound of every in-kernel wait; 0 = default (4000) */
  int32_t device;                   /* CUDA device ordinal, -1 = current */
  int32_t max_tokens_per_request;   /* prompt tokens one request may be fed per iteration (the reference's
                                       MPK_MAX_TOKENS_PER_REQUEST, persistent_kernel.cuh:443-449); 0 = as many as
                                       the iteration's token budget max_num_batched_tokens allows */
  /* ---- measurement and test aids: not part of the operator API.  Leave them zero in
   * production; mk_create warns on stderr when debug_flags is set, because it changes results. */
  int32_t trace_op;                 /* device op whose inner phases are stamped into the profiler buffer (stored +1: 0 = none) */
  int32_t debug_flags;              /* bit 0: linear tasks skip the arithmetic (weight-stream timing only); bit 1: attention tasks keep their barrier and do nothing else.  RESULTS ARE WRONG with either bit.  bit 4: no tagged activations: every op of the row-owner path keeps its grid barrier (results unchanged) */
  int32_t max_stages;               /* cap on the weight ring depth, 0 = default */
  int32_t prefetch_kb;              /* KB of weights per CTA requested into L2 ahead of the shared-memory ring; 0 = default (512 for a row-owner program that keeps its grid barriers, off otherwise), < 0 = off */
  int32_t cluster_size;             /* CTAs per thread-block cluster of the launch: 0 = default, 1 = flat grid barrier, 2 or 4 = hierarchical (cluster-first) grid barrier */
  uint32_t test_barrier_epoch;      /* tests only: barrier epoch every launch starts at (e.g. just below the 32-bit wrap of the counter) */
  int32_t reserved[2];
} mk_config;

/* PersistentKernel.__init__ -> KNGraph(CyKNGraph(...)) (persistent_kernel.py:404). */
mk_handle* mk_create(const mk_config* cfg);

/* attach_input (persistent_kernel.py:469-480; core.pyx attach_torch_tensor):
 * borrow a caller-owned, row-major device tensor.  Returns the tensor id. */
int mk_tensor_attach(mk_handle* h, const char* name, void* device_ptr, int dtype, int ndim, const int64_t* dims,
                     const int64_t* strides);

/* new_tensor (persistent_kernel.py:482-503; attach_cuda_tensor / attach_nvshmem_tensor):
 * a runtime-owned intermediate.  strides may be NULL (row-major). */
int mk_tensor_new(mk_handle* h, const char* name, int dtype, int ndim, const int64_t* dims, const int64_t* strides,
                  int category);

/* shuffle_tensors (persistent_kernel.py:513-519; python/mirage/mpk/models/utils.py:40-118):
 * rows of the inputs interleaved in num_groups groups, materialised at compile time. */
int mk_tensor_shuffle(mk_handle* h, const char* name, const int* tensor_ids, int n, int shuffled_dim, int num_groups);

/* fuse_tensors (persistent_kernel.py:505-511): same as shuffle with the inputs concatenated per group. */
int mk_tensor_fuse(mk_handle* h, const char* name, const int* tensor_ids, int n, int fused_dim, int num_groups);

/* kn_graph.customized + register_task (core.pyx:944-1013; src/kernel/graph.cc:439-848).
 * op_name is the layer's task family: "embedding", "rmsnorm", "rmsnorm_linear",
 * "linear", "linear_with_residual", "paged_attention", "paged_attention_split_kv",
 * "paged_attention_split_kv_merge", "silu_mul", "argmax", "argmax_partial",
 * "argmax_reduce", "allreduce" (params: num_gpus, my_gpu_id).  tensor_ids are the layer's operands in the
 * order the Python method lists them; params are its integer parameters. */
int mk_op(mk_handle* h, const char* op_name, const int* tensor_ids, int n_tensors, const int64_t* params, int n_params,
          const int* grid_dim, const int* block_dim);

/* Meta tensors of the constructor (persistent_kernel.py:417-452), device pointers in
 * this order: step, tokens, input_tokens, output_tokens, num_new_tokens,
 * prompt_lengths, qo_indptr_buffer, paged_kv_indptr_buffer,
 * paged_kv_indices_buffer, paged_kv_last_page_len_buffer.
 * Stands in for init_func (persistent_kernel.py:35) / init_persistent_kernel
 * (persistent_kernel.cuh:1966). */
int mk_set_meta(mk_handle* h, void* const meta_ptrs[10], int64_t total_num_requests, void* profiler_ptr);

/* profiler_tensor of the constructor (persistent_kernel.py:361-362, profiler.h:116-181): a
 * caller-owned uint64 device buffer of n_entries words.  When set before mk_compile, the
 * kernel leaves a trace of the LAST iteration in it: word [(op * grid + cta) * 4 + k] is the
 * globaltimer (ns) at which CTA `cta` reached device op `op` (k=0), passed its barrier (k=1)
 * and finished it (k=2); op == mk_num_device_ops() is the iteration prologue. */
int mk_set_profiler(mk_handle* h, void* device_ptr, int64_t n_entries);

/* compile (persistent_kernel.py:2404-2618; generate_task_graph, src/kernel/runtime.cc:1652):
 * validates the graph, lowers it to the device program, materialises shuffled
 * weights, encodes TMA descriptors and allocates scratch.  No JIT. */
int mk_compile(mk_handle* h);

/* init_request_func / init_request_resources (persistent_kernel.cuh:1960):
 * reset step[], the request slots and the page free list. */
int mk_init_requests(mk_handle* h, void* stream);

/* launch_func / launch_persistent_kernel (persistent_kernel.cuh:2260): run the whole
 * generation (offline) or one pass (onepass) and wait for it.  Returns MK_E_DEVICE
 * if the kernel raised its abort flag. */
int mk_launch(mk_handle* h, void* stream);
/* Same, without waiting; pair with mk_wait. */
int mk_launch_async(mk_handle* h, void* stream);
int mk_wait(mk_handle* h, void* stream);

/* get_event_timing_func (persistent_kernel.cuh:2412): per-iteration records of the
 * last launch as pairs (globaltimer ns at iteration start, active tokens).
 * Returns the number of iterations copied. */
int mk_get_event_timing(mk_handle* h, uint64_t* host_buf, int max_entries);

/* finalize_func / finalize_persistent_kernel (persistent_kernel.cuh:2331). */
int mk_finalize(mk_handle* h);

int mk_last_error(mk_handle* h, char* buf, int n);

/* Tensor parallelism.  The reference puts its activation buffers on the NVSHMEM symmetric heap
 * (persistent_kernel.cuh:1921-1938, 2002-2015) and exchanges 128-byte slices with
 * nvshmemx_putmem_signal_block (src/kernel/task_register.cc:1649-1673).  Here each rank (one
 * process per GPU) owns one exchange region; the in-kernel allreduce stores straight into the
 * peers' regions over NVLink.  mk_comm_prepare plans the graph, allocates the region and writes
 * its 64-byte CUDA IPC handle (returns 1; 0 when the graph needs no exchange); the caller
 * gathers the handles of all ranks (any transport: torch.distributed, MPI, files) and passes
 * them, ordered by rank, to mk_comm_connect; then mk_compile.  All ranks must launch together. */
int mk_comm_prepare(mk_handle* h, unsigned char handle_out[64]);
int mk_comm_connect(mk_handle* h, const unsigned char* handles /* world_size x 64 */, int n);

/* Host-only half of mk_compile (validation, fusion decisions, device-op list); needs no GPU. */
int mk_plan(mk_handle* h);

/* Introspection used by the host-side tests and the benchmark. */
int mk_num_device_ops(mk_handle* h);
int mk_describe(mk_handle* h, char* buf, int n);       /* one line per device op */
int mk_grid_size(mk_handle* h);
int64_t mk_weight_bytes_per_step(mk_handle* h);        /* bytes the TMA producer streams per iteration */
int mk_debug_partition(int64_t nblk, int64_t nkt, int grid, int64_t* begin_out /* grid+1 */, int* owner_check);
/* The arithmetic of the tensor-parallel exchange and of the grid barrier, as the device does it
 * (used by the host-side tests).  Exchange k (1-based) of a launch that follows total_before
 * completed exchanges: its number, the first 8-byte word of its half of a region, and how many of
 * the numbers a slot may still hold from earlier uses would be taken for "arrived" (must be 0). */
int mk_debug_exchange_sequence(uint32_t total_before, uint32_t k, int world, int tokens, int cols, uint32_t* seq_out,
                               int64_t* first_word_out, int* stale_arrived_out);
int mk_barrier_target_reached(uint32_t counter, uint32_t epoch, uint32_t arrivals_per_barrier);
void* mk_tensor_ptr(mk_handle* h, int tensor_id);      /* device address after compile (runtime-owned ones too) */
int mk_tensor_read(mk_handle* h, int tensor_id, void* host_buf, int64_t bytes); /* copy a tensor's bytes to the host */

/* No counterpart in the reference (its runtime allocates everything it needs).
 *
 * A linear layer for hosts that cannot allocate device memory where they need it: a server
 * that gave the whole GPU to its own arena at start-up, or a loop that must not run into
 * the device-wide synchronisation of cudaMalloc / cudaFree.  Computes
 *     out[t][j] = bf16( sum_i x[t][i] * w[j][i]  (+ residual[t][j]) ),   fp32 accumulation,
 * for row-major bf16 x [tokens, k], w [n, k], residual (may be NULL) and out [tokens, n],
 * all caller-owned device memory, 16-byte aligned, k a multiple of 8.  The call allocates
 * and frees nothing: the partial sums of its k-splits live in a fixed array inside the
 * library (about 4 MB on every GPU that loads it, held until the process exits), which is
 * why the sizes are capped: tokens <= MK_STATIC_MAX_TOKENS, n <= MK_STATIC_MAX_N,
 * k <= MK_STATIC_MAX_K; anything larger returns MK_E_TOO_LARGE (and says so on stderr).
 * The first call on a device looks up that array's device address; make this first call
 * outside any stream capture.  All calls share the array: calls that overlap on the GPU
 * race on it, so issue them on one stream or otherwise serialise them.  The launch is
 * asynchronous on `stream`; the return value covers argument checks and launch errors.
 * Not thread-safe: the per-device address cache and the scratch are shared by all callers. */
#define MK_STATIC_MAX_TOKENS 8
#define MK_STATIC_MAX_N 16384
#define MK_STATIC_MAX_K 32768
int mk_linear_static(const void* x, const void* w, const void* residual, void* out, int tokens, int n, int k,
                     void* stream);

#ifdef __cplusplus
}
#endif
#endif
