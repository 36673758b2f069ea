// Shared host/device definitions of the B200 decode megakernel.
//
// The host runtime lowers the recorded operator list into a flat array of
// OpDesc (the "program").  One persistent cooperative kernel walks that array
// once per decode iteration on every SM.
#pragma once
#include <stdint.h>

namespace mk {

// ---- geometry of the weight stream -------------------------------------------------
// A weight tile is 128 output rows x 128 k-elements of bf16 (32 KB): two 2-D TMA boxes
// of 128 rows x 64 k-elements, adjacent in k, each landing 128-byte-swizzled in its half
// of a shared-memory stage.  One mbarrier round trip per 32 KB keeps the producer and
// consumer loops off the critical path.
constexpr int kTileRows = 128;
constexpr int kBoxK = 64;                         // k-elements of one TMA box (128 bytes: the swizzle span)
constexpr int kSubTiles = 2;                      // boxes per stage, adjacent in k
constexpr int kTileK = kBoxK * kSubTiles;         // k-elements per stage
constexpr int kSubBytes = kTileRows * kBoxK * 2;  // 16 KB
constexpr int kStageBytes = kSubBytes * kSubTiles;
constexpr int kNumConsumerWarps = 8;
constexpr int kNumConsumers = kNumConsumerWarps * 32;
constexpr int kNumThreads = kNumConsumers + 64;  // + the weight producer warp and the activation producer warp
constexpr int kMaxTokGroup = 8;                  // tokens per pass of a linear op (one mma n-tile)
constexpr int kHeadDim = 128;
// Row-owner linear (one or two batched tokens): a CTA owns a contiguous range of 8-row units
// and walks it in chunks of up to 32 rows; a stage holds a chunk's rows for 512 k-elements
// as eight TMA boxes of 64 k-elements (32 KB for a full chunk).
constexpr int kUnitRows = 8;
constexpr int kChunkRows = 32;
constexpr int kRowsStageK = 512;

enum OpType : int {
  OP_EMBED = 1,
  OP_RMSNORM = 2,
  OP_LINEAR = 3,
  OP_ATTN = 4,
  OP_SILU_MUL = 5,
  OP_ARGMAX_PARTIAL = 6,
  OP_ARGMAX_REDUCE = 7,
  OP_ALLREDUCE = 8,
  // mixture of experts (one or two batched tokens: every (token, expert slot) pair is a row-owner GEMV)
  OP_MOE_ROUTE = 9,    // router logits [T, experts] -> top-k expert ids and renormalised softmax weights
  OP_MOE_LINEAR = 10,  // out[pair] = W[expert of the pair] * in[token or pair]; n = rows per expert, aux1 = experts
  OP_MOE_COMBINE = 11, // out[t] = sum over the token's slots of weight * in[pair] (+ residual)
};

enum OpFlags : int {
  F_SYNC_BEFORE = 1 << 0,   // grid barrier before the op
  F_CTA0_ONLY = 1 << 1,     // only CTA 0 executes the body
  F_NORM_IN = 1 << 2,       // linear: RMSNorm fused on the input rows
  F_RESIDUAL = 1 << 3,      // linear: + residual
  F_SILU_MUL = 1 << 4,      // linear: rows are [64 gate | 64 up] per tile, epilogue SiLU(gate)*up
  F_ARGMAX = 1 << 5,        // linear: per-tile (max, index) of the bf16 logits
  F_QK_NORM = 1 << 6,       // attention
  F_ROPE = 1 << 7,          // attention
  F_WRITE_NORM = 1 << 8,    // linear with F_NORM_IN: CTA 0 also stores the normalised rows
  F_RES_RANK0 = 1 << 9,     // residual only contributed when rank == 0 (row-parallel TP)
  F_XTILE = 1 << 10,        // linear: input rows arrive per stage by TMA as activation boxes
  F_ROWS = 1 << 11,         // linear: every CTA owns whole output rows (no split over k between CTAs)
  // tensor parallelism: the allreduce behind a row-parallel linear folded into its neighbours
  F_PUSH = 1 << 12,         // linear: the epilogue stores its fp32 sums into every rank's exchange slots instead of `out`
  F_GATHER_IN = 1 << 13,    // linear / rmsnorm: the input rows are the rank-order sum of the latest exchange's slots
  F_GATHER_RES = 1 << 14,   // linear: the residual is the rank-order sum of the latest exchange's slots
  F_MOE_PAIR_IN = 1 << 17,  // MoE linear: the input has one row per (token, slot) pair (the down projection), not one per token
  F_XRANK = 1 << 16,        // argmax reduce: the per-rank (value, index) pairs of a vocabulary-sharded LM head are exchanged and the global best is taken
  F_SILU4 = 1 << 15,        // linear with F_SILU_MUL on the tile paths: rows are [4 gate | 4 up] per 8-row unit (the row-owner layout)
  // Tagged activations (row-owner path): a producer also stores its bf16 outputs as 8-byte words
  // {two adjacent columns, tag of the producing op in this iteration}; a consumer polls the words
  // it needs instead of waiting at a grid barrier, so data and "ready" arrive in one load.
  F_LL_OUT = 1 << 18,       // linear / attention: the outputs are also stored as tagged words (ll_out)
  F_LL_IN = 1 << 19,        // linear / attention: the input rows are read from tagged words (ll_in, producer op ll_in_op); no barrier
  F_LL_RES = 1 << 20,       // linear: the residual is read from tagged words (ll_res, producer op ll_res_op)
  F_MOE_COMBINE = 1 << 23,  // MoE down linear: a CTA owns output rows for ALL expert slots of a token and adds the slots up itself
                            // (weights amax_val, + res), out: [T, n]; no per-slot output, no separate weighted-sum op
  F_MOE_ROUTE = 1 << 22,    // MoE gate/up linear: the op first routes the tokens itself (res: router logits [T, experts]); every CTA
                            // keeps the expert ids in shared memory for its producer, CTA 0 also stores the runtime's tables
  F_XRED = 1 << 21,         // linear with F_LL_IN under tensor parallelism: the op first adds up its slice of the latest exchange
                            // over the ranks and stores it as tagged words (ll_in, tagged as its own output), then reads them all
};

enum Numerics : int {
  NUM_MPK = 0,    // fp32 task arithmetic of the reference megakernel, one bf16 rounding per task
  NUM_TORCH = 1,  // bf16 roundings of the reference PyTorch model (no-eps bf16 RMSNorm, ...)
};

enum Mode : int { MODE_OFFLINE = 0, MODE_ONEPASS = 1 };

// The kernel is compiled once per linear-layer path, each instance holding only the code its
// path runs: the whole step executes out of the instruction cache once per layer, and code
// that is merely present (other paths' loops) measurably slowed the batch-1 step down.
enum Path : int {
  PATH_ROWS = 0,   // 1-2 tokens: row-owner linears, resident token rows, L2 look-ahead
  PATH_TILES = 1,  // 3-16 tokens (and graphs the row-owner path cannot take): stream-K tiles, mma.sync
  PATH_UMMA = 2,   // 17-64 tokens: stream-K tiles, tcgen05.mma, grouped attention
};

enum Status : int {
  ST_OK = 0,
  ST_TIMEOUT_GRID = 1,
  ST_TIMEOUT_FULL = 2,
  ST_TIMEOUT_EMPTY = 3,
  ST_TIMEOUT_GO = 4,
  ST_TIMEOUT_PEER = 5,
  ST_BAD_TOKEN = 6,
  ST_OUT_OF_PAGES = 7,
  ST_TIMEOUT_RANK = 8,
  ST_TIMEOUT_DATA = 9,
};

struct alignas(16) OpDesc {
  int type;
  int flags;
  // generic shapes
  int n;        // linear: output features; rmsnorm/silu: columns; argmax: vocab
  int k;        // linear: input features
  int ld_in, ld_out, ld_res, ld_out2;  // row pitches in elements
  int nblk, nkt;                       // linear: row tiles, k tiles (F_ROWS: nkt = 512-wide k stages)
  int aux0, aux1, aux2, aux3;          // per-type small ints (see mk_kernel.cu)
  const void* in;
  const void* w;       // linear weight / embedding table / rmsnorm weight
  const void* norm_w;  // fused input norm weight
  const void* res;
  void* out;
  void* out2;
  const void* tmap_w;  // device address of the CUtensorMap of w
  // attention
  const void* tmap_x;     // linear, wide batches: device address of the CUtensorMap of the input rows
  void* k_cache;
  void* v_cache;
  const void* q_norm_w;
  const void* k_norm_w;
  const void* cos;
  const void* sin;
  // argmax partials
  float* amax_val;
  int* amax_idx;
  int amax_n;   // number of partials per token
  int pad_;
  // tagged activations: word (token t, column pair j) of a tensor with row pitch ld sits at [t * (ld / 2) + j]
  const void* ll_in;
  void* ll_out;
  const void* ll_res;
  int ll_in_op, ll_res_op;  // program indices of the ops that produce ll_in / ll_res
};

struct KParams {
  const OpDesc* ops;
  int num_ops;
  int mode;
  int path;  // Path: which instance of the kernel the host launches
  int numerics;
  int rank, world;
  // meta tensors of the operator API (caller-owned)
  int* step;
  long long* tokens;
  long long* input_tokens;
  long long* output_tokens;
  int* num_new_tokens;
  int* prompt_lengths;
  int* qo_indptr;
  int* kv_indptr;
  int* kv_indices;
  int* kv_last_page_len;
  int max_seq_len, max_reqs, max_tokens, max_pages, page_size, total_requests;
  int max_tokens_per_req;  // prompt tokens one request may get per iteration (chunked prefill)
  // A handle may hold two programs over the same state: one planned for iterations of at most
  // max_reqs tokens (decode) and one for the larger iterations that carry prompt chunks.  A launch
  // serves iterations of tok_lo .. tok_hi tokens and hands any other to the host, which launches
  // the other program (ctrl[0] = -2, the prepared token count in sched[5]).
  int tok_lo, tok_hi;
  int page_shift;  // log2(page_size): page sizes are powers of two
  long long eos;
  int vocab_limit;  // embedding rows, to refuse out-of-range token ids
  // runtime-owned state
  int* request_ids;   // [max_reqs]
  int* page_queue;    // ring of free pages [max_pages]
  int* sched;         // [0]=page head [1]=page tail [2]=next request id [3]=iterations done
                      // [4]=outputs of the last iteration not appended yet
                      // [5]=tokens of an iteration that is prepared but was handed to the other program
                      // [6]=exchanges executed by the last launch
                      // [7]=iterations completed by earlier kernels of the current generation call
  unsigned* grid_bar;
  int cluster;            // CTAs per thread-block cluster of the launch (1 = flat grid barrier)
  unsigned bar_epoch0;    // barrier epoch the launch starts at (the counter is preset to match; tests start near the wrap)
  int* ctrl;          // [0] = active tokens of the iteration, -1 = terminate, -2 = hand over to the other program
  int* abort_flag;
  int* status;        // [0]=code [1]=cta [2]=op [3]=iter [4..7]=detail
  unsigned long long* step_times;
  int max_step_times;
  int max_iters;      // 0 = unlimited
  unsigned long long timeout_ns;
  // split-k scratch shared by all linear ops
  float* partial;         // [groups][grid][2][128*kMaxTokGroup]
  unsigned* piece_count;  // [groups][max nblk]
  int piece_stride;       // max nblk
  // attention scratch
  float* attn_part;       // [tokens][kv heads][max chunks][qpk*(128+2)]
  unsigned* attn_count;   // [tokens][kv heads]
  int attn_max_chunks;
  uint2* attn_part_ll;    // the same partials as tagged 8-byte words {fp32, tag}, for the merge without a counter (null: not used)
  // tensor-parallel exchange: every rank's exchange region mapped into this GPU's address space
  // (xchg[rank] is the local one).  A region holds slots [2][world][xchg_tokens][xchg_cols] of 8-byte
  // words {fp32 value, sequence number}: a word is valid for exchange number s once its second half
  // equals s, so data and "arrived" flag travel in one store and no fence or separate flag is needed.
  // Exchange s uses the half of the region selected by s & 1 (see xchg_word).
  unsigned char* xchg[8];
  int xchg_tokens, xchg_cols;
  // behind the slots: [world][xchg_tokens][2] words {logit value, number} {vocabulary index, number} for the
  // argmax of a vocabulary-sharded LM head (one buffer: a rank cannot be a whole iteration ahead of a peer)
  long long xchg_amax_word;  // index of that area, in 8-byte words
  unsigned xchg_seq_base;  // exchanges executed by all earlier launches: sequence numbers keep growing (mod 2^32)
  // optional per-op trace of the last iteration: [(op * grid + cta) * 4 + k] globaltimer ns,
  // k = 0 op reached, 1 barrier passed, 2 op done; op == num_ops is the iteration prologue
  unsigned long long* prof;
  int trace_op;     // op whose inner phases are stamped: prof[(num_ops + 1) * grid * 4 + cta * 16 + k]; -1 none
  int debug_flags;  // bit 0: linear tasks skip the arithmetic
  int prefetch_tiles;  // weight tiles per CTA requested into L2 ahead of the ring (0 = off)
  int has_moe;         // the program holds mixture-of-experts ops: the host launches the build of the kernel that has them
  // shared-memory carve-up (bytes from the 1024-aligned base)
  int num_stages;
  int stage_bytes;  // weights (kStageBytes) + the activation boxes of a wide-batch stage
  int x_rows;       // token rows of an activation box (0: activations are staged by the consumers)
  int sums_off;     // per-(row, token) sums of a run of tiles: [128][sums_stride] floats
  int sums_stride;
  int x_off, x_bytes;
  int red_off;
  int bar_off;
};

// Exchange sequence arithmetic (shared with the host-side checks).  Exchange k (1-based) of a launch
// that follows `total_before` completed exchanges has number total_before + k, modulo 2^32; number 0 is
// skipped by nobody: a word is "arrived" only when it carries exactly the awaited number, and the
// previous occupants of a slot carry numbers that differ from it by a multiple of 2 up to the region's
// age, so a collision needs 2^32 exchanges between two uses of one slot.
__host__ __device__ inline unsigned xchg_seq(unsigned total_before, unsigned k) { return total_before + k; }
__host__ __device__ inline unsigned xchg_half(unsigned seq) { return seq & 1u; }
__host__ __device__ inline bool xchg_arrived(unsigned word_seq, unsigned seq) { return word_seq == seq; }
// index (in 8-byte words) of (exchange seq, source rank, token row, column) in a region
__host__ __device__ inline size_t xchg_word(unsigned seq, int world, int tokens, int cols, int src, int tok, int col) {
  return (((size_t)xchg_half(seq) * world + src) * tokens + tok) * cols + col;
}

// Tag of the words op `op` stores in iteration `iter` (1-based) of a launch.  The host clears the word
// buffers before every launch, and tags grow with (iteration, op), so a buffer never holds the awaited
// tag before its producer in this iteration has stored it.
__host__ __device__ inline unsigned ll_tag(int iter, int num_ops, int op) {
  return (unsigned)(iter - 1) * (unsigned)num_ops + (unsigned)op + 1u;
}

// Weight tiles of a linear op are dealt to `grid` CTAs as contiguous ranges
// [c*total/grid, (c+1)*total/grid); tile_owner is the inverse.  32-bit arithmetic: the
// host refuses ops with total * (grid + 1) >= 2^32 tiles.
__host__ __device__ inline unsigned tile_begin(unsigned c, unsigned total, unsigned grid) {
  return c * total / grid;
}
__host__ __device__ inline int tile_owner(unsigned tile, unsigned total, unsigned grid) {
  return (int)(((tile + 1u) * grid - 1u) / total);
}

static_assert(sizeof(OpDesc) % 16 == 0 && sizeof(OpDesc) <= 256, "OpDesc is copied to shared memory in 16-byte pieces");

}  // namespace mk
