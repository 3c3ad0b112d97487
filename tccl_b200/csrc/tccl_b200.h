/*
 * C ABI of libtccl_b200: hand-written sm_100a collectives over peer-mapped
 * (symmetric) memory.  Everything here is plain C so that the library can be
 * loaded with ctypes / dlopen and carries no dependency on libtorch.
 *
 * Conventions
 *  - Every launcher enqueues exactly one kernel on `stream` and returns the
 *    cudaError_t of the launch (0 = success) or a negative TCCL_E* code for an
 *    argument the launcher rejects.  Nothing synchronises the host.
 *  - "real" mode (n_emu == 0): `comm` / `args` point to ONE struct in host
 *    memory describing the calling rank.
 *  - "emulated" mode (n_emu == W >= 1): `comm` / `args` point to arrays of W
 *    structs in DEVICE memory; one cooperative launch with gridDim.y == W runs
 *    all W ranks on the current GPU (blockIdx.y is the rank).  This is how the
 *    multi-rank protocols are exercised on a single GPU.
 *  - Device-side waits are bounded by `timeout_ns`; a wait that runs out
 *    records a status (see tccl_status_word) and the kernel returns.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCCL_MAX_WORLD 8

/* flag-region layout (in 32-bit words, per rank); the region is zeroed by reset */
#define TCCL_MAX_BLOCKS 1024                                     /* barrier rows */
#define TCCL_FLAG_BAR 0                                          /* [block][src]          */
#define TCCL_FLAG_MCBAR (TCCL_FLAG_BAR + TCCL_MAX_BLOCKS * TCCL_MAX_WORLD) /* [block]     */
#define TCCL_FLAG_TREE_UP (TCCL_FLAG_MCBAR + TCCL_MAX_BLOCKS)    /* [tree][cta][2 slots]  */
#define TCCL_TREE_MAX_CTAS 128
#define TCCL_FLAG_TREE_DOWN (TCCL_FLAG_TREE_UP + 2 * TCCL_TREE_MAX_CTAS * 2) /* [tree][cta] */
#define TCCL_FLAG_TILE (TCCL_FLAG_TREE_DOWN + 2 * TCCL_TREE_MAX_CTAS)  /* [src][tile] GEMM */
#define TCCL_MAX_TILES 4096
#define TCCL_FLAG_LL (TCCL_FLAG_TILE + TCCL_MAX_WORLD * TCCL_MAX_TILES) /* misc / p2p */
#define TCCL_FLAG_AG (TCCL_FLAG_LL + 1024)                            /* [src][row tile] AG->GEMM */
#define TCCL_MAX_ROW_TILES 256
#define TCCL_FLAG_TREE_ACK (TCCL_FLAG_AG + TCCL_MAX_WORLD * TCCL_MAX_ROW_TILES) /* [tree][cta]: my chunks the parent has consumed */
#define TCCL_FLAG_TREE_DACK (TCCL_FLAG_TREE_ACK + 2 * TCCL_TREE_MAX_CTAS) /* [tree][cta][2 slots]: slices a child has pulled */
#define TCCL_FLAG_WORDS (TCCL_FLAG_TREE_DACK + 2 * TCCL_TREE_MAX_CTAS * 2)

/* local (non peer-visible) state, in 32-bit words */
#define TCCL_LOCAL_EPOCH 0                                       /* [block] p2p barrier   */
#define TCCL_LOCAL_MCEPOCH (TCCL_LOCAL_EPOCH + TCCL_MAX_BLOCKS)  /* [block] nvls barrier  */
#define TCCL_LOCAL_STATUS (TCCL_LOCAL_MCEPOCH + TCCL_MAX_BLOCKS) /* tccl_status_word      */
#define TCCL_LOCAL_TILE_EPOCH (TCCL_LOCAL_STATUS + 16)           /* 1 word: tile epoch    */
#define TCCL_LOCAL_SCHED (TCCL_LOCAL_TILE_EPOCH + 1)             /* [0] CTAs of a fused kernel that are done */
#define TCCL_LOCAL_AGCNT (TCCL_LOCAL_SCHED + 63)                 /* [row tile] data movers done (AG->GEMM) */
#define TCCL_LOCAL_PUSH_SEQ (TCCL_LOCAL_AGCNT + TCCL_MAX_ROW_TILES) /* push all-reduce calls completed (slot parity) */
#define TCCL_LOCAL_PUSH_DONE (TCCL_LOCAL_PUSH_SEQ + 1)           /* CTAs of the running push all-reduce that are done */
#define TCCL_LOCAL_TREE_SEQ (TCCL_LOCAL_PUSH_DONE + 1)           /* [role][cta]: chunks this pipeline moved in earlier calls */
#define TCCL_LOCAL_RS_SEQ (TCCL_LOCAL_TREE_SEQ + 4 * TCCL_TREE_MAX_CTAS) /* pair GEMM -> RS calls completed (staging half) */
#define TCCL_LOCAL_RS_NEXT (TCCL_LOCAL_RS_SEQ + 1)               /* pair GEMM -> RS: next reduction unit to hand out */
#define TCCL_LOCAL_AG_SEQ (TCCL_LOCAL_RS_NEXT + 1)               /* pair AG -> GEMM calls completed (gather buffer half) */
#define TCCL_LOCAL_TREE_LL_SEQ (TCCL_LOCAL_AG_SEQ + 1)            /* [role][cta]: calls of the small-message tree kernel */
#define TCCL_LOCAL_WORDS (TCCL_LOCAL_TREE_LL_SEQ + 4 * 32)

enum tccl_status_word {
  TCCL_ST_CODE = 0,   /* 0 = ok, else tccl_error */
  TCCL_ST_BLOCK = 1,  /* blockIdx.x of the first waiter that gave up */
  TCCL_ST_PEER = 2,   /* peer rank it was waiting for */
  TCCL_ST_WHERE = 3,  /* tccl_where */
  TCCL_ST_SEEN = 4,   /* flag value last seen */
  TCCL_ST_WANT = 5,   /* flag value waited for */
  TCCL_ST_ABORT = 6,  /* non-zero: all further waits of this rank return at once */
  TCCL_ST_WORDS = 16
};

enum tccl_error { TCCL_OK = 0, TCCL_TIMEOUT = 1, TCCL_BAD_INDEX = 2 };
enum tccl_where {
  TCCL_W_BARRIER = 1, TCCL_W_MCBARRIER = 2, TCCL_W_CAS_SEND = 3, TCCL_W_CAS_WAIT = 4,
  TCCL_W_TREE_UP = 5, TCCL_W_TREE_DOWN = 6, TCCL_W_TILE = 7, TCCL_W_SIGNAL = 8,
  TCCL_W_MBAR = 9,
  TCCL_W_INDEX_IN = 10, TCCL_W_INDEX_OUT = 11 /* TCCL_BAD_INDEX: an input / output offset beyond its extent */
};

/* launcher-side argument errors (returned negated) */
enum tccl_arg_error { TCCL_EINVAL = 1000, TCCL_EDTYPE = 1001, TCCL_EALIGN = 1002, TCCL_ESIZE = 1003 };

enum tccl_dtype { TCCL_BF16 = 0, TCCL_F32 = 1, TCCL_F16 = 2 };

/* One rank's view of the communicator.  All pointers are device addresses. */
typedef struct tccl_comm {
  int32_t world;
  int32_t rank;
  uint32_t* flags[TCCL_MAX_WORLD]; /* every rank's flag region, peer-mapped */
  uint32_t* mc_flags;              /* multicast alias of the flag region, or NULL */
  uint32_t* local;                 /* this rank's private state (TCCL_LOCAL_*) */
  char* stage[TCCL_MAX_WORLD];     /* every rank's staging area, peer-mapped */
  char* mc_stage;                  /* multicast alias of the staging area, or NULL */
  uint64_t stage_bytes;            /* bytes of the staging area the fused kernels may use */
  uint64_t timeout_ns;
  uint64_t ll_bytes;               /* bytes of the small-message region that follows: stage[p] + stage_bytes */
  uint64_t tree_bytes;             /* bytes of the double-tree ring that follows the small-message region */
} tccl_comm;

/* double-tree ring.  First the small-message (flag-in-line) part: slots [tree][left, right, down][cta][seq % depth];
 * of TCCL_TREE_LL_SLOT_BYTES each; then the chunked part: slots [tree][child slot][cta][chunk % depth] of
 * TCCL_TREE_SLICE_BYTES each (large slices: the cost of a slice's flag traffic and release fence is per slice). */
#define TCCL_TREE_SLICE_BYTES 262144
#define TCCL_TREE_LL_SLOT_BYTES 65536
#define TCCL_TREE_RING_DEPTH 4
#define TCCL_TREE_LL_MAX_CTAS 32
#define TCCL_TREE_LL_BYTES (2 * 3 * TCCL_TREE_LL_MAX_CTAS * TCCL_TREE_RING_DEPTH * TCCL_TREE_LL_SLOT_BYTES)

/* Arguments shared by the data collectives. */
typedef struct tccl_coll_args {
  const void* in[TCCL_MAX_WORLD]; /* every rank's input (peer-mapped, view offset applied) */
  void* mc_in;                    /* multicast alias of the input, or NULL */
  void* out;                      /* local output (may be NULL for in-place variants) */
  void* out_peer[TCCL_MAX_WORLD]; /* every rank's output when it is symmetric, else unused */
  void* mc_out;                   /* multicast alias of the symmetric output, or NULL */
  uint64_t numel;                 /* elements of the per-rank input */
  int32_t dtype;                  /* tccl_dtype */
  int32_t flags;                  /* TCCL_F_* */
  uint64_t in_bytes;              /* bytes that may be read from every in[p] / mc_in ... */
  uint64_t out_bytes;             /* ... and written at out / every out_peer[p] / mc_out: checked by the
                                     TCCL_DEBUG_CHECKS build of the library, ignored by the regular one */
} tccl_coll_args;

#define TCCL_F_NO_EXIT_BARRIER 1 /* caller guarantees inputs stay untouched until peers are done */
#define TCCL_F_NO_ENTRY_BARRIER 2
#define TCCL_F_NVLS_BARRIER 4    /* use the multimem.red barrier flavour */
/* pipelined two-shot all-reduce only; the same bits go into tccl_launch.meta */
#define TCCL_F_PIPE_REDUCERS_SHIFT 8  /* 4 bits: warps (of 16) that pull; the others push */
#define TCCL_F_PIPE_STAGES_SHIFT 12   /* 4 bits: shared-memory stages - 1 */
#define TCCL_F_PIPE_UNROLL_SHIFT 16   /* 4 bits: vectors per reducer thread per stage (2, 4 or 8) */

typedef struct tccl_launch {
  int32_t grid;    /* CTAs per rank */
  int32_t block;   /* threads per CTA */
  int32_t n_emu;   /* 0 = real, W = emulate W ranks on this GPU */
  int32_t meta;    /* bits 0-7: tccl_dtype of the args (read in emulated mode, where they are device-resident);
                      bits 8..: kernel-specific shape bits (TCCL_F_PIPE_*) */
  void* stream;    /* cudaStream_t */
} tccl_launch;

int tccl_version(void);
/* 1 if this library was built with TCCL_DEBUG_CHECKS (every vector offset of the flat collectives is
 * checked against the extents in tccl_coll_args; a miss records TCCL_BAD_INDEX and skips the access) */
int tccl_debug_checks(void);
const char* tccl_error_string(int code);
int tccl_num_sms(void);
/* sizeof of an ABI struct by its name ("tccl_comm", ...), -1 if unknown */
int tccl_sizeof(const char* name);

/* ---- barriers -------------------------------------------------------- */
typedef struct tccl_barrier_args {
  int32_t rounds; /* barrier rounds to run back to back inside one launch */
} tccl_barrier_args;
typedef struct tccl_pads_args {
  uint32_t* pads[TCCL_MAX_WORLD]; /* every rank's signal pad, peer-mapped, laid out [block][world] */
} tccl_pads_args;
/* epoch barrier on the library's own flag region, by posted stores to every peer */
int tccl_barrier_p2p(const tccl_comm*, const tccl_barrier_args*, const tccl_launch*);
/* same, one multimem.red through the switch instead of W stores (needs comm->mc_flags) */
int tccl_barrier_nvls(const tccl_comm*, const tccl_barrier_args*, const tccl_launch*);
/* self-resetting CAS barrier on caller-provided signal pads (the layout of torch
 * symmetric memory's signal pads) */
int tccl_barrier_cas(const tccl_comm*, const tccl_pads_args*, const tccl_launch*);
/* waits for a flag that nothing sets: exercises the timeout path (tests only) */
int tccl_wait_never(const tccl_comm*, const tccl_barrier_args*, const tccl_launch*);

/* ---- data collectives ------------------------------------------------- */
int tccl_allreduce_oneshot_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allreduce_oneshot_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
/* small-message latency path: push into the peers' staging slots, one barrier, local sum.
 * The slots live in the small-message region of the communicator (comm->stage[p] + comm->stage_bytes,
 * comm->ll_bytes long): two halves used alternately from call to call, each cut into `world` slots of
 * tccl_push_slot_bytes() whatever the message size.  in[rank] = the local input (any device
 * memory); numel * sizeof(T) % 16 == 0 and at most one slot. */
uint64_t tccl_push_slot_bytes(uint64_t ll_bytes, int world);
int tccl_allreduce_push_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allreduce_push_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allreduce_twoshot_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allreduce_twoshot_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
/* two-shot with reducer and broadcaster warps decoupled through a shared-memory ring (block = 512) */
int tccl_allreduce_twoshot_pipe_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allreduce_twoshot_pipe_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
/* Two-shot all-reduce that moves the data with bulk async copies (global -> shared -> global; no thread touches
 * remote memory).  l->block must be 256; dynamic shared memory is (3 * world + 2) * tccl_allreduce_bulk_chunk_bytes(). */
uint32_t tccl_allreduce_bulk_chunk_bytes(int world);
int tccl_allreduce_twoshot_bulk(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allgather_pull_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allgather_push_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_allgather_push_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_reducescatter_p2p(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);
int tccl_reducescatter_nvls(const tccl_comm*, const tccl_coll_args*, const tccl_launch*);

/* ---- double-binary-tree all-reduce --------------------------------------- */
typedef struct tccl_tree_args {
  const void* in;            /* this rank's input: any device memory; may be buf[rank] (in place) */
  void* buf[TCCL_MAX_WORLD]; /* every rank's result buffer (symmetric): parents store the sum into their children's */
  void* out;                 /* optional local copy of the result in ordinary memory, or NULL */
  uint64_t numel;            /* a whole number of 16-byte vectors */
  uint64_t chunk_vecs;       /* 16-byte vectors per chunk (<= ctas_per_role * TCCL_TREE_SLICE_BYTES / 16); chunk c uses tree c % 2 */
  int32_t dtype;
  int32_t ctas_per_role;     /* K; the grid is 4 K CTAs (up/down x tree 0/1); K <= tccl_tree_max_ctas(comm->tree_bytes) */
  int32_t parent[2];         /* neighbours in tree 0 / 1, -1 = none */
  int32_t left[2];
  int32_t right[2];
  int32_t child_slot[2];     /* 0 if this rank is its parent's left child, 1 if right */
} tccl_tree_args;
/* TCCL_TREE_PULL_DOWN in l->meta: on the way down the children load the sum from their parent's result
 * buffer instead of the parent storing it into theirs (buf must then be readable by the children until they
 * have acknowledged, which the kernel waits for); measured slower than pushing, so off by default */
#define TCCL_TREE_PULL_DOWN 256
int tccl_allreduce_tree(const tccl_comm*, const tccl_tree_args*, const tccl_launch*);
/* CTAs per role that a ring of `tree_bytes` can serve (<= TCCL_TREE_MAX_CTAS) */
int tccl_tree_max_ctas(uint64_t tree_bytes);
/* Small messages: every 16-byte line on the wire carries 8 bytes of data and the call's sequence number
 * twice, so a hop needs neither a release nor a counter.  numel * sizeof(T) <= 2 * ctas_per_role * 32 KiB,
 * ctas_per_role <= TCCL_TREE_LL_MAX_CTAS.  Of args->buf only buf[rank] is used (this rank's own result
 * buffer; may be null); nothing has to be in symmetric memory. */
int tccl_allreduce_tree_ll(const tccl_comm*, const tccl_tree_args*, const tccl_launch*);

/* ---- all-reduce with a quantised wire format ------------------------------- */
typedef struct tccl_qar_args {
  const void* in;   /* this rank's bf16 input, any device memory */
  void* out;        /* this rank's bf16 output (may be `in`) */
  uint64_t numel;   /* a multiple of 2048 */
  int32_t flags;    /* reserved, 0 */
} tccl_qar_args;
/* bytes of staging area (per rank) the kernel needs */
uint64_t tccl_allreduce_fp8wire_stage_bytes(uint64_t numel, int world);
/* fp8 (e4m3) + one fp32 scale per 2048 elements on the wire, fp32 accumulation at the owner; l->block == 256 */
int tccl_allreduce_fp8wire(const tccl_comm*, const tccl_qar_args*, const tccl_launch*);

/* ---- fused all-reduce + bias + residual + RMSNorm ------------------------- */
typedef struct tccl_arn_args {
  const void* x[TCCL_MAX_WORLD];   /* every rank's partial [tokens, hidden] (symmetric, peer-mapped) */
  void* mc_x;                      /* multicast alias of x, or NULL */
  void* out[TCCL_MAX_WORLD];       /* every rank's normalised output (symmetric) */
  void* mc_out;
  void* res_out[TCCL_MAX_WORLD];   /* every rank's pre-norm sum (symmetric), or all NULL to skip it */
  void* mc_res_out;
  const void* bias;                /* [hidden] or NULL */
  const void* residual;            /* local [tokens, hidden] or NULL */
  const void* weight;              /* [hidden] */
  float eps;
  int32_t tokens, hidden;          /* hidden * sizeof(T) % 16 == 0, hidden <= 2048 * (16 / sizeof(T)) */
  int32_t dtype;
  int32_t flags;                   /* TCCL_F_NVLS_BARRIER */
} tccl_arn_args;
/* `hidden` repeats args->hidden for the host (in emulated mode `args` is a device pointer) */
int tccl_allreduce_bias_residual_rmsnorm(const tccl_comm*, const tccl_arn_args*, int nvls, int hidden,
                                         const tccl_launch*);

/* ---- tcgen05 GEMM (bf16 in, fp32 accumulate in tensor memory, bf16 out) ---- */
typedef struct tccl_gemm_args {
  const void* a;   /* [m, k], k contiguous, lda elements between rows */
  const void* bt;  /* [n, k], k contiguous (the layout of a torch Linear weight) */
  void* c;         /* [m, n] */
  void* status;    /* optional: TCCL_ST_WORDS uint32 words for a timeout report, or NULL */
  int32_t m, n, k;
  int32_t lda, ldb, ldc;
} tccl_gemm_args;
/* c = a * bt^T on this GPU; grid <= 0 picks one CTA per SM */
int tccl_gemm_bf16(const tccl_gemm_args*, int grid, void* stream);
/* same product on pairs of CTAs (tcgen05.mma.cta_group::2): 256 x 256 tiles, each CTA loads its own
 * 128 rows of a and its own half of bt; the last partial wave is cut into 256 x 128 half tiles */
int tccl_gemm_bf16_pair(const tccl_gemm_args*, int grid, void* stream);

/* ---- fused GEMM -> reduce-scatter (rows scattered over the ranks) ---------- */
typedef struct tccl_gemm_rs_args {
  const void* a;   /* this rank's [m, k] activations (its K-slice), k contiguous */
  const void* bt;  /* this rank's [n, k] weight slice, k contiguous */
  void* out;       /* this rank's [m / world, n] result rows */
  int32_t m, n, k; /* m % (world * 128) == 0, n % 256 == 0, k % 8 == 0 */
  int32_t lda, ldb, ldo;
  void* trace;     /* optional: grid * 64 uint64 words of per-tile %globaltimer stamps, or NULL */
} tccl_gemm_rs_args;
/* bytes of staging area (per rank) the fused kernel needs for an m x n product */
uint64_t tccl_gemm_rs_stage_bytes(int m, int n, int world);
uint64_t tccl_gemm_rs_param_bytes(void);
/* real mode: comm/args are host structs, dev_params unused.  Emulated mode: comm is the
 * device array of communicators, args a HOST array of n_emu structs, dev_params device
 * scratch of n_emu * tccl_gemm_rs_param_bytes() bytes (64-byte aligned). */
int tccl_gemm_reduce_scatter(const tccl_comm* comm, const tccl_gemm_rs_args* args, void* dev_params,
                             uint64_t stage_bytes, const tccl_launch* l);

/* Same product on CTA pairs (tcgen05.mma.cta_group::2), tiles interleaved over the owners so that the
 * reduction overlaps the mainloop, and no entry barrier: the staging area is used in two alternating
 * halves.  m % (world * 256) == 0; l->grid even.  TCCL_RS_SYNC_ENTRY in l->meta asks for an entry
 * barrier (needed when the previous user of the staging area was another kernel). */
#define TCCL_RS_SYNC_ENTRY 256
uint64_t tccl_gemm_rs_pair_stage_bytes(int m, int n, int world);
uint64_t tccl_gemm_rs_pair_param_bytes(void);
int tccl_gemm_reduce_scatter_pair(const tccl_comm* comm, const tccl_gemm_rs_args* args, void* dev_params,
                                  uint64_t stage_bytes, const tccl_launch* l);

/* ---- fused all-gather -> GEMM (rows gathered over the ranks) -------------- */
typedef struct tccl_ag_gemm_args {
  const void* a_shard;              /* this rank's [m / world, k] rows, k contiguous */
  void* a_full[TCCL_MAX_WORLD];     /* every rank's gathered [m, k] buffer (symmetric, peer-mapped) */
  void* mc_a_full;                  /* multicast alias of the gathered buffer, or NULL */
  const void* bt;                   /* this rank's [n, k] weight slice, k contiguous */
  void* out;                        /* this rank's [m, n] result */
  int32_t m, n, k;                  /* m % (world * 128) == 0, n % 8 == 0, k % 8 == 0 */
  int32_t lda_shard, lda_full, ldb, ldo;
  int32_t comm_ctas;                /* CTAs that move the shard; the others run the GEMM */
  int32_t swiglu;                   /* 1: every 256-row block of bt is 128 gate rows then the 128 matching up
                                       rows; out is [m, n / 2] = silu(gate) * up (n % 256 == 0) */
  void* trace;                      /* optional: grid * 64 uint64 words of per-tile %globaltimer stamps */
  int32_t lsu_movers;               /* 1: move the shard with LSU / multimem.st stores instead of bulk copies */
  int32_t sched_stride;             /* pair kernel: entries per CTA pair in `sched` */
  const int32_t* sched;             /* pair kernel, optional (device memory): the tiles of every CTA pair in the order
                                       it runs them, [pairs][sched_stride] entries TCCL_AG_UNIT(mt, nt, half), ended
                                       by -1; mt = even 128-row tile, half = 0 (256 columns) / 1 / 2 (left / right
                                       128).  NULL: own rows first, then the peers' rows in arrival order */
} tccl_ag_gemm_args;
#define TCCL_AG_UNIT(mt, nt, half) ((int32_t)(mt) | ((int32_t)(nt) << 12) | ((int32_t)(half) << 28))
uint64_t tccl_ag_gemm_param_bytes(void);
/* same calling convention as tccl_gemm_reduce_scatter */
int tccl_allgather_gemm(const tccl_comm* comm, const tccl_ag_gemm_args* args, void* dev_params,
                        const tccl_launch* l);

/* Same product on CTA pairs (tcgen05.mma.cta_group::2); every CTA moves its share of the shard first
 * (comm_ctas = batches of that phase, 0 = 2; lsu_movers bit 2 = move only, bit 4 = send destination by
 * destination with plain stores instead of batch by batch to all ranks).  m % (world * 256) == 0; l->grid even.  `half_bytes`: distance
 * from a_full[q] to the second half of every rank's gathered buffer — the halves alternate from call to
 * call and no entry barrier is needed — or 0 for a single buffer (the kernel then opens with a barrier). */
uint64_t tccl_ag_gemm_pair_param_bytes(void);
int tccl_allgather_gemm_pair(const tccl_comm* comm, const tccl_ag_gemm_args* args, void* dev_params,
                             uint64_t half_bytes, const tccl_launch* l);

#ifdef __cplusplus
}
#endif
