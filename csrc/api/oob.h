/* C ABI of the library (loaded from Python with ctypes, usable from C/C++).
 *
 * Capability parity: the reference's include/ooverlap/comm.h:54-358
 * (oo_group_* / oo_node_* / oo_buffer_* / oo_ipc_slot_set_* / oo_allreduce* /
 * oo_reduce_scatter* / oo_all_gather*).  The object model is collapsed to one
 * communicator per rank process that owns a symmetric heap: every rank maps
 * every other rank's heap (and, where the driver allows, an NVLink multicast
 * alias of all of them), so a buffer is identified by (registration id,
 * byte offset) and no per-call exchange is ever needed.
 *
 * All functions return 0 on success or a negative oob_status_t; the message of
 * the last failure on the calling thread is available from oob_last_error().
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

typedef struct oob_comm oob_comm;

typedef enum {
  OOB_OK = 0,
  OOB_ERR_INVALID = -1,
  OOB_ERR_CUDA = -2,
  OOB_ERR_BOOTSTRAP = -3,
  OOB_ERR_UNSUPPORTED = -4,
  OOB_ERR_NOMEM = -5,
  OOB_ERR_DEVICE_TIMEOUT = -6, /* a kernel gave up waiting; see oob_comm_status */
  OOB_ERR_POISONED = -7        /* an earlier device timeout left the flags inconsistent */
} oob_status_t;

typedef enum { OOB_F16 = 0, OOB_BF16 = 1, OOB_F32 = 2 } oob_dtype_t;
typedef enum { OOB_SUM = 0, OOB_MIN = 1, OOB_MAX = 2 } oob_op_t;

/* Algorithms; OOB_ALGO_AUTO asks the tuning policy. */
#define OOB_ALGO_AUTO (-1)
typedef enum { OOB_AR_ONESHOT_P2P = 0, OOB_AR_TWOSHOT_P2P = 1, OOB_AR_TWOSHOT_NVLS = 2, OOB_AR_ONESHOT_NVLS = 3 } oob_ar_algo_t;
typedef enum { OOB_RS_P2P = 0, OOB_RS_NVLS = 1 } oob_rs_algo_t;
typedef enum { OOB_AG_PUSH_P2P = 0, OOB_AG_PUSH_NVLS = 1, OOB_AG_PULL_P2P = 2 } oob_ag_algo_t;
typedef enum {
  OOB_NORM_LOCAL = 0,
  OOB_NORM_AR_ONESHOT = 1,
  OOB_NORM_AR_TWOSHOT = 2,
  OOB_NORM_AR_TWOSHOT_NVLS = 3,
  OOB_NORM_RS = 4,
  OOB_NORM_RS_NVLS = 5,
  OOB_NORM_AR_PUSH = 6,      /* decode sizes: push + one barrier + local sum and norm of every row; needs stage_* */
  OOB_NORM_AR_PUSH_NVLS = 7,
  OOB_NORM_AR_LL = 8         /* the smallest messages: 8-byte cells of data + call number, no barrier; stage_* names the
                                zeroed staging area of oob_allreduce_ll, piece_bytes >= 2 x the message */
} oob_norm_algo_t;
typedef enum { OOB_GEMM_PLAIN = 0, OOB_GEMM_AR = 1, OOB_GEMM_RS_NORM = 2, OOB_GEMM_AG = 3 } oob_gemm_mode_t;

/* Creation flags */
#define OOB_FLAG_NO_NVLS 1u        /* never create a multicast object */
#define OOB_FLAG_LEGACY_IPC 2u     /* cudaMalloc + cudaIpc handles instead of VMM file descriptors */

typedef struct {
  int rank, world, device;
  int nvls;            /* 1 when the heap has a multicast alias */
  int emulated;        /* 1 for the single-GPU emulation group */
  int memory_kind;     /* 0 = VMM fd, 1 = legacy IPC, 2 = same-process */
  uint64_t heap_bytes; /* per rank, including the signal pad */
  uint64_t user_offset;/* first byte available to oob_alloc */
  uint64_t timeout_ns;
} oob_comm_info_t;

typedef struct {
  int code, rank, peer, block;
  unsigned expected, observed;
  int where, pad;
} oob_device_status_t;

const char* oob_last_error(void);
/* Logging of the native runtime: level 0 error, 1 warn (default), 2 info, 3 debug; OOB_LOG_LEVEL sets it from the
 * environment.  Records go to stderr unless a sink is installed (the sink may be called from any thread). */
typedef void (*oob_log_sink_t)(int level, const char* message);
int oob_set_log_level(int level);
int oob_get_log_level(void);
int oob_set_log_sink(oob_log_sink_t sink);
int oob_log_message(int level, const char* message);
const char* oob_version(void);

/* One call per rank process.  `key` names the rendezvous (<= 80 chars). */
int oob_comm_create(int rank, int world, int device, const char* key, uint64_t heap_bytes, unsigned flags,
                    int timeout_ms, oob_comm** out);
/* All `world` ranks live in this process on `device`; collectives are run as
 * ONE cooperative launch whose block rows act as ranks.  For tests and tuning
 * on a single GPU. */
int oob_comm_create_emulated(int world, int device, uint64_t heap_bytes, oob_comm** out);
int oob_comm_destroy(oob_comm* c);
int oob_comm_info(const oob_comm* c, oob_comm_info_t* info);
int oob_comm_set_timeout_ms(oob_comm* c, int ms);
int oob_comm_barrier(oob_comm* c);                       /* host-side, through the rendezvous */
/* Host-side all-gather of `bytes` bytes per rank through the rendezvous (out holds world x bytes, in rank order).  Works
 * while the device side is poisoned, so ranks can agree on what to do after a device timeout. */
int oob_comm_host_allgather(oob_comm* c, const void* in, void* out, uint64_t bytes);
int oob_comm_status(oob_comm* c, oob_device_status_t* s);/* 0 = clean, OOB_ERR_DEVICE_TIMEOUT otherwise */
/* Collective: zeroes every rank's signal pad and status after a device
 * timeout.  No kernel of this communicator may be in flight. */
int oob_comm_recover(oob_comm* c);

/* Symmetric heap.  Every rank must issue the same sequence of alloc/free
 * calls; offsets are then identical on all ranks. */
int oob_alloc(oob_comm* c, uint64_t bytes, uint64_t align, uint64_t* offset);
int oob_free(oob_comm* c, uint64_t offset);
void* oob_heap_ptr(const oob_comm* c, int rank, uint64_t offset);
void* oob_heap_mc_ptr(const oob_comm* c, uint64_t offset);

/* Registers memory that was NOT allocated from the heap (e.g. a torch tensor)
 * through legacy CUDA IPC: the allocation's base is shared once and kept in an
 * import cache, the view is base + offset.  Collective.  Returns the
 * registration id (> 0) in *reg. */
int oob_register_ipc(oob_comm* c, void* ptr, uint64_t bytes, int* reg);
int oob_unregister(oob_comm* c, int reg);

/* Buffers are (reg, offset): reg 0 is the heap. */
int oob_allreduce(oob_comm* c, int dtype, int op, int algo, int in_reg, uint64_t in_off, int out_reg, uint64_t out_off,
                  void* out_local, uint64_t count, int max_ctas, void* stream);
int oob_reduce_scatter(oob_comm* c, int dtype, int op, int algo, int in_reg, uint64_t in_off, void* out_local,
                       uint64_t count, int max_ctas, void* stream);
int oob_all_gather(oob_comm* c, int dtype, int algo, int out_reg, uint64_t out_off, const void* src_local,
                   void* dst_local, uint64_t count, int max_ctas, void* stream);

/* Small-message all-reduce with ONE rank barrier and no separate copy: `in_local` (any device memory, `count`
 * elements) is pushed into piece `rank` of the registered staging area (stage_reg, stage_off) on every rank, the ranks
 * meet once, and every rank sums the pieces from its own memory in rank order (fp32) into `out_local` (any device
 * memory; may alias in_local).  The staging area holds TWO sets of world * piece_bytes bytes (piece_bytes a multiple
 * of 16 and >= the message); consecutive calls alternate between the sets, decided by a call counter on the device,
 * so calls may follow one another at once, also as replays of captured graphs.  Only this entry point may write to
 * the staging area, and every rank must make the same sequence of calls.  use_nvls != 0 pushes with multimem.st when
 * the heap has a multicast alias.  Moves (world - 1) x the message per rank: for messages up to a few hundred KiB. */
int oob_allreduce_push(oob_comm* c, int dtype, int op, int stage_reg, uint64_t stage_off, uint64_t piece_bytes,
                       const void* in_local, void* out_local, uint64_t count, int use_nvls, int max_ctas, void* stream);
/* The lowest-latency all-reduce, for messages of a few KiB to a few tens of KiB: no barrier and no fence.  Every rank
 * stores its input into its piece of the staging area on all ranks as 8-byte cells {4 data bytes, 4 flag bytes = number
 * of this call}; receivers spin on the cells and sum them in rank order (fp32) into `out_local`.  The staging area
 * (stage_reg, stage_off) holds TWO sets of world * piece_bytes bytes, piece_bytes a multiple of 16 and at least 8 bytes
 * per 32-bit word of the message.  It must be zeroed on every rank before the first call (with a host barrier after
 * the zeroing) and again before oob_comm_recover (which restarts the call numbers), and nothing but this entry point
 * may write to it.  Every rank must make the same sequence of calls. */
int oob_allreduce_ll(oob_comm* c, int dtype, int op, int stage_reg, uint64_t stage_off, uint64_t piece_bytes,
                     const void* in_local, void* out_local, uint64_t count, int use_nvls, int max_ctas, void* stream);

/* All-to-all: `src_local` holds `world` chunks of count_per_peer elements; chunk j goes to rank j and lands as
 * chunk (this rank) of its registered output buffer (world * count_per_peer elements).  No counterpart in the
 * reference (it only has an NCCL send/recv baseline). */
int oob_all_to_all(oob_comm* c, int dtype, int out_reg, uint64_t out_off, const void* src_local, uint64_t count_per_peer,
                   int max_ctas, void* stream);

typedef struct {
  int dtype, rows, hidden;
  float eps;
  int x_reg;
  uint64_t x_off;
  const void* residual;
  const void* weight;
  int y_reg;
  uint64_t y_off; /* two-shot algorithms: y in registered memory */
  void* y_local;  /* other algorithms */
  int res_out_reg;
  uint64_t res_out_off; /* reg < 0: no residual output */
  void* res_out_local;
  uint64_t emu_stride_local; /* emulation: byte stride between ranks of residual / y_local / res_out_local */
  int stage_reg;             /* push algorithms: staging area of the push kernels (see oob_allreduce_push): two sets of */
  uint64_t stage_off;        /* world * piece_bytes; outputs are y_local / res_out_local                                */
  uint64_t piece_bytes;
} oob_norm_args_t;
int oob_fused_norm(oob_comm* c, int algo, const oob_norm_args_t* a, int max_ctas, void* stream);

typedef struct {
  int mode, dtype;
  int M, N, K;
  const void* A;
  int lda;
  const void* B;
  int ldb;
  void* C;
  int ldc;
  uint64_t a_emu_stride, b_emu_stride, c_emu_stride;
  int comm_ctas, max_ctas;
  int partial_reg;
  uint64_t partial_off;
  int c_reg;
  uint64_t c_off;
  int counter_base;
  const void* residual;
  const void* weight;
  float eps;
  void* y_local;
  void* res_out_local;
  uint64_t rs_emu_stride;
  int a_full_reg;
  uint64_t a_full_off;
  int use_nvls; /* fused modes: 0 = peer loads/stores only, non-zero = NVLS multimem when the heap has it */
  int splits;   /* plain mode: K splits per tile; 0 = chosen from the shape, 1 = off */
  int no_join;  /* fused AR / RS: 1 = only the dedicated communication CTAs reduce */
  void* trace;  /* optional device buffer, 8 x uint64 per CTA: globaltimer stamps of the kernel's phases */
  int pair;     /* 0 = two-SM kernel (CTA pairs, 256x256 tiles) when the shape suits it, 1 = whenever possible,
                   -1 = never; plain and fused modes (fused GEMM->AR on pairs reduces C in place and ignores partial_*) */
  int splitk_reduce; /* split-K: 0 / 1 = separate reduction kernel, -1 = sum inside the GEMM kernel */
  int skinny;   /* plain mode, M <= 128: 1 = weight-streaming stream-K kernel; 0 / -1 = tiled kernels */
  int epilogue; /* plain mode, split problems only (oob_gemm_plan_splits > 1): OOB_EPILOGUE_* applied by the kernel
                   that sums the K splits */
  const void* epilogue_args; /* host pointer: oob_gemm_epilogue_swiglu_t or oob_rope_args_t (oob_model.h) */
  int gemv;     /* plain mode, M <= 4: 1 = CUDA-core streaming kernel, 0 = by shape (M = 1; M = 2 with N x K <= 12 M),
                   -1 = never */
  int stream_k; /* two-SM kernel, plain and AG modes: stream-K tail; 0 = when it pays for the shape, 1 = whenever the
                   tile count leaves a remainder, -1 = never */
  void* order;  /* two-SM kernel: optional device buffer, 2 x uint64 per 128-row half of every 256x256 tile (index
                   2 * tile's number in the schedule + CTA of the pair): [0] globaltimer ns at which the half was
                   complete (fused AR / RS: published to its reducer), [1] = pair << 32 | index in the pair's sequence */
} oob_gemm_args_t;
#define OOB_EPILOGUE_NONE 0
#define OOB_EPILOGUE_SWIGLU 1  /* N = 2F columns [gate | up]; C is [M, F] = silu(gate) * up */
#define OOB_EPILOGUE_ROPE_KV 2 /* columns = (H + 2 KV) heads of hd: rotate q and k, q -> q_out, k and v -> cache; C unused */
typedef struct {
  int F;
} oob_gemm_epilogue_swiglu_t;
/* Number of K splits oob_gemm uses for a plain GEMM of this shape (`splits` as in oob_gemm_args_t, 0 = by shape). */
int oob_gemm_plan_splits(int M, int N, int K, int max_ctas, int splits);
/* c may be NULL for OOB_GEMM_PLAIN. */
int oob_gemm(oob_comm* c, const oob_gemm_args_t* a, void* stream);
int oob_gemm_counters_needed(int mode, int M, int N, int world);
/* Allocates, on the current device, the scratch memory that later oob_gemm calls would otherwise allocate on first
 * use: the stream-K workspace of the two-SM kernel (fixed size) and a split-K workspace of at least splitk_bytes
 * (0 = none; see oob_gemm_splitk_bytes).  Call it before capturing a CUDA graph: an allocation cannot happen during
 * capture, and oob_gemm then fails with OOB_ERR_UNSUPPORTED instead of growing the workspace.  Workspaces handed
 * out earlier are never freed or moved, so graphs that were captured with them stay valid. */
int oob_gemm_reserve_workspace(uint64_t splitk_bytes);
/* Split-K workspace bytes a plain GEMM of this shape needs (0 when it is not split). */
uint64_t oob_gemm_splitk_bytes(int M, int N, int K, int max_ctas, int splits);
uint64_t oob_gemm_partial_bytes(int M, int N);

/* Tuning policy (size -> algorithm, CTA budget). */
int oob_policy_load(const char* json_path);
int oob_policy_select(int world, int collective /*0 AR,1 RS,2 AG*/, uint64_t bytes, int nvls, int* algo, int* ctas);

/* Topology probe; writes a JSON document into buf (truncated to cap). */
int oob_topology_json(char* buf, uint64_t cap, int run_probes);
/* The same document with every switch: `flags` is a mask of OOB_TOPO_*, `devices` lists the device indices to describe
 * (NULL / 0 = all visible ones).  OOB_TOPO_TEXT writes a table instead of JSON.  With OOB_TOPO_REQUIRE_PEER the call
 * fails with OOB_ERR_UNSUPPORTED (the message names the pairs) when a listed pair has no peer access. */
#define OOB_TOPO_PROBES 1u            /* live probes: remote ld/st, remote atomic, timed peer copy, multimem */
#define OOB_TOPO_NO_ENABLE_PEER 2u    /* never switch peer access on (the per-pair probes are then skipped) */
#define OOB_TOPO_NO_ATOMIC_PROBE 4u
#define OOB_TOPO_NO_COPY_PROBE 8u
#define OOB_TOPO_NO_MULTIMEM_PROBE 16u
#define OOB_TOPO_REQUIRE_PEER 32u
#define OOB_TOPO_TEXT 64u
#define OOB_TOPO_NO_BULK_PROBE 128u   /* skip the bulk-store (cp.async.bulk shared -> peer global) probe */
int oob_topology_describe(char* buf, uint64_t cap, unsigned flags, const int* devices, int n_devices);

/* Node-local rendezvous on its own (host only): all-gather of small blobs,
 * barrier, file-descriptor exchange.  Every call has the creation timeout. */
typedef struct oob_bootstrap oob_bootstrap;
int oob_bootstrap_create(int rank, int world, const char* key, int timeout_ms, oob_bootstrap** out);
int oob_bootstrap_destroy(oob_bootstrap* h);
int oob_bootstrap_allgather(oob_bootstrap* h, const void* in, void* out, uint64_t bytes);
int oob_bootstrap_barrier(oob_bootstrap* h);
int oob_bootstrap_exchange_fds(oob_bootstrap* h, int my_fd, int* fds_out /* world entries */);
int oob_bootstrap_broadcast_fd(oob_bootstrap* h, int root, int* fd);

/* Byte offset (inside every rank's heap) and number of the general arrival counters of the signal pad, for tools
 * that verify that an op left them re-armed (all zero between launches). */
uint64_t oob_pad_counter_offset(void);
int oob_pad_counter_count(void);

/* Test hook (host only): work items of the two-SM GEMM's schedule for a problem on `pairs` CTA pairs, nine integers
 * per item: pair, schedule position, m block, n block, first K block, end K block, stream-K workspace slot (-1 for
 * whole tiles, -2 for the part that starts a tile: its pair owns the tile and parks nothing), parts of the tile, first
 * pair of the tile.  Returns the item count, -1 when cap is too small. */
int oob_test_pair_schedule(int mode, int M, int N, int K, int pairs, int stream_k, int world, int rank, int* out, int cap);

/* Test hook: waits on a flag that nobody sets, with the communicator's
 * timeout, and reports through the status block (bounded-wait self test). */
int oob_test_bounded_wait(oob_comm* c, void* stream);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
