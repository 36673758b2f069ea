// Host runtime behind the C ABI: records the operator list, lowers it to the
// device program (fusing RMSNorm, SiLU*up and the argmax partials into the
// linear tasks where the intermediate is runtime-owned and has one reader),
// materialises shuffled weights, encodes TMA descriptors, owns scratch and
// launches the persistent kernel.
//
// Stands in for the reference's Cython binding + task-graph compiler + JIT
// (python/mirage/_cython/core.pyx:944-1013, src/kernel/graph.cc:338-848,
// src/kernel/runtime.cc:53-1685, python/mirage/mpk/persistent_kernel.py:2404-2618)
// and its host launcher (include/mirage/persistent_kernel/persistent_kernel.cuh:1960-2429).
// There is no code generation: the kernel is compiled ahead of time and reads
// shapes from the program.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/b200mk.h"
#include "mk_types.h"

extern "C" int mk_kernel_max_ctas_per_sm(const mk::KParams* p, int smem_bytes);
extern "C" int mk_kernel_max_clusters(int path, int smem_bytes, int cluster, int grid);
extern "C" int mk_kernel_launch(const mk::KParams* p, int grid, int smem_bytes, void* stream);
extern "C" int mk_kernel_init_state(const mk::KParams* p, void* stream);

namespace {

constexpr int kMaxSmem = 232448;  // 227 KB opt-in limit per CTA on sm_100
constexpr int kRedBytes = 2048;    // small scratch (reductions, argmax, sequence lengths)
constexpr int kFastSmem = 166912;  // 164 KB carve-out minus the 1 KB the system reserves per CTA
constexpr int kRowsSumsBytes = mk::kNumConsumerWarps * mk::kChunkRows * 2 * 4;  // [warp][32 rows][2 tokens] floats
// token rows a row-owner CTA may keep resident beside three 32 KB weight stages
constexpr int kRowsXBudget = kFastSmem - 2048 - kRedBytes - kRowsSumsBytes - 3 * mk::kStageBytes;
constexpr int kAttnMaxChunks = 32;
constexpr int kMaxStepTimes = 16384;

size_t dtype_size(int dt) {
  switch (dt) {
    case MK_BF16: case MK_F16: return 2;
    case MK_F32: case MK_I32: return 4;
    default: return 8;
  }
}

struct Tensor {
  std::string name;
  int dtype = MK_BF16;
  int ndim = 0;
  int64_t dims[4] = {1, 1, 1, 1};
  int64_t strides[4] = {1, 1, 1, 1};
  void* ptr = nullptr;
  bool owned = false;       // allocated by the runtime
  bool user = false;        // attached by the caller: contents are observable
  std::vector<int> src;     // shuffle/fuse sources
  int groups = 0;
  int interleave = 0;  // > 0: two sources laid out as [g rows of src0 | g rows of src1] repeating (g = 64 or 4)
  int readers = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= dims[i];
    return n;
  }
  size_t alloc_bytes() const {
    int64_t m = 1;
    for (int i = 0; i < ndim; ++i) m = std::max<int64_t>(m, dims[i] * strides[i]);
    return (size_t)m * dtype_size(dtype);
  }
};

struct RecOp {
  std::string name;
  std::vector<int> t;
  std::vector<int64_t> params;
  int grid[3] = {1, 1, 1};
  int block[3] = {1, 1, 1};
};

// A device op before addresses are known: tensor ids instead of pointers.
struct PlanOp {
  int type = 0, flags = 0;
  int in = -1, w = -1, norm_w = -1, res = -1, out = -1;
  int kc = -1, vc = -1, qn = -1, kn = -1, cos = -1, sin = -1;
  int n = 0, k = 0, aux0 = 0, aux1 = 0, aux2 = 0, aux3 = 0;
  int amax_n = 0;
  int ll_in_op = -1, ll_res_op = -1;  // tagged activations: the ops that produce the input / the residual
  std::string note;
};

bool starts_with(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }
bool canonical_name_is_w2(const std::string& s) { return starts_with(s, "moe_w2_linear") || s == "gang_moe_w2"; }

}  // namespace

// A lowered program and what was built for it.  A handle holds one, or two over the same
// tensors and scheduler state: the primary one, planned for iterations of at most
// max_num_batched_requests tokens (every request decoding), and, where prompt chunks make
// iterations wider than that and the width puts the linears on another path, a second one
// planned for max_num_batched_tokens.  The persistent kernel hands an iteration that is not
// for its program back to the host, which launches the other one (see mk_wait).
struct Program {
  std::vector<PlanOp> plan;
  bool rows_mode = false;
  int max_tokens = 0;  // widest iteration it is planned for
  mk::KParams kp{};
  int smem_bytes = 0;
  int64_t weight_bytes = 0;
  int max_nblk = 1;
  size_t attn_count_bytes = 0, piece_count_bytes = 0;  // arrival counters, cleared before every kernel launch
  void* ll_buf = nullptr;  // tagged activation words of the program, cleared before every kernel launch
  size_t ll_bytes = 0;
};

struct mk_handle {
  mk_config cfg{};
  std::vector<Tensor> tensors;
  std::vector<RecOp> ops;    // layers as recorded
  std::vector<RecOp> nops;   // the same with aliases of one device op folded onto its plain name
  std::vector<PlanOp> plan;
  bool planned = false, compiled = false, meta_set = false;
  bool rows_mode = false;  // linear layers run row-owner (F_ROWS)
  // plan / rows_mode / kp / smem_bytes / weight_bytes / max_nblk above and below are the program being
  // built or, after compile, a copy of the primary program (what the introspection calls describe)
  Program prog[2];
  int nprog = 0;
  int cur_prog = 0;          // program the next kernel of a launch uses
  int plan_tokens = 0;       // widest iteration the plan being built must serve
  int force_interleave = 0;  // gate/up weight layout fixed by the primary program (4 or 64), 0 = the plan's own choice
  std::string err;
  void* meta[10] = {};
  int64_t total_requests = 0;
  int num_sms = 0;
  int grid = 0, smem_bytes = 0;
  mk::KParams kp{};
  std::vector<void*> allocs;
  int max_nblk = 1;
  int64_t weight_bytes = 0;
  bool launched = false;
  void* prof_ptr = nullptr;
  int64_t prof_entries = 0;
  // tensor-parallel exchange
  void* xchg_local = nullptr;
  void* xchg_peer[8] = {};
  bool xchg_ready = false;
  int xchg_tokens = 0, xchg_cols = 0;
  long long xchg_amax_word = 0;
  unsigned xchg_total = 0;      // cross-rank exchanges executed by all completed launches (all ranks advance alike)
  bool in_flight = false;       // launched and not yet waited for
  bool poisoned = false;        // a tensor-parallel launch aborted: the ranks' exchange sequences may differ
  size_t attn_count_bytes = 0;  // the attention chunk counters, cleared before every launch
  size_t piece_count_bytes = 0; // the split-k arrival counters, cleared before every launch
  void* ll_buf = nullptr;       // tagged activation words of the program being compiled
  size_t ll_bytes = 0;

  int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    err = buf;
    return code;
  }
  int cuda_fail(cudaError_t e, const char* what) {
    return fail(MK_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  int dmalloc(void** p, size_t bytes, bool zero = true) {
    cudaError_t e = cudaMalloc(p, std::max<size_t>(bytes, 256));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc");
    allocs.push_back(*p);
    if (zero) {
      e = cudaMemset(*p, 0, std::max<size_t>(bytes, 256));
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemset");
    }
    return 0;
  }
};

namespace {

bool valid_tensor(mk_handle* h, int id) { return id >= 0 && id < (int)h->tensors.size(); }

int add_tensor(mk_handle* h, const char* name, int dtype, int ndim, const int64_t* dims, const int64_t* strides) {
  if (!name || ndim < 1 || ndim > 4 || !dims) return h->fail(MK_E_INVALID, "tensor needs a name and 1..4 dims");
  if (dtype < MK_BF16 || dtype > MK_F16) return h->fail(MK_E_INVALID, "tensor %s: unknown dtype %d", name, dtype);
  Tensor t;
  t.name = name;
  t.dtype = dtype;
  t.ndim = ndim;
  int64_t s = 1;
  for (int i = ndim - 1; i >= 0; --i) {
    if (dims[i] <= 0) return h->fail(MK_E_INVALID, "tensor %s: dim %d is %lld", name, i, (long long)dims[i]);
    t.dims[i] = dims[i];
    t.strides[i] = strides ? strides[i] : s;
    s *= dims[i];
  }
  h->tensors.push_back(t);
  return (int)h->tensors.size() - 1;
}

// ------------------------------------------------------------------------------------
// lowering: recorded layers -> device ops (host only, no CUDA calls)
// ------------------------------------------------------------------------------------
bool is_linear(const std::string& n) {
  return n == "linear" || starts_with(n, "linear_sm100") || n == "linear_with_residual" ||
         starts_with(n, "linear_with_residual_sm100") || starts_with(n, "linear_swapAB") || n == "rmsnorm_linear" ||
         n == "linear_silu" || n == "splitk_linear" || n == "silu_mul_linear_with_residual";
}

int check_2d_bf16(mk_handle* h, int id, const char* what) {
  const Tensor& t = h->tensors[id];
  if (t.ndim != 2 || t.dtype != MK_BF16)
    return h->fail(MK_E_INVALID, "%s: tensor %s must be 2-D bf16", what, t.name.c_str());
  if (t.strides[1] != 1) return h->fail(MK_E_INVALID, "%s: tensor %s must be row-major", what, t.name.c_str());
  return 0;
}

// The reference registers many task names for one operator: per-architecture variants
// (linear_sm100, rmsnorm_hopper, ...) and Fleet's gang_* family, whose extra arguments
// (tile_n, m_tiles, wgm, k_splits, workspaces, done counters) describe ITS tiling
// (python/mirage/mpk/persistent_kernel.py:1064-2043).  Here the tiling is the runtime's own
// choice, so every alias folds onto the plain layer: same operands minus the scratch ones.
RecOp canonical_op(const RecOp& in) {
  RecOp op = in;
  const std::string& n = in.name;
  auto keep = [&](std::initializer_list<int> idx) {
    std::vector<int> t;
    for (int i : idx)
      if (i < (int)in.t.size()) t.push_back(in.t[i]);
    op.t = t;
  };
  if (starts_with(n, "gang_rmsnorm")) {
    op.name = "rmsnorm";
  } else if (starts_with(n, "gang_linear_silu") || starts_with(n, "linear_silu")) {
    op.name = "linear_silu";
  } else if (starts_with(n, "gang_linear_res") || starts_with(n, "linear_with_residual_m_parallel")) {
    op.name = "linear_with_residual";  // (input, weight, residual, output)
  } else if (starts_with(n, "gang_ksplit_") || starts_with(n, "gang_splitk_linear_res")) {
    op.name = "linear_with_residual";  // (input, weight, residual, workspace, output)
    keep({0, 1, 2, 4});
  } else if (starts_with(n, "splitk_linear_res_atomic")) {
    op.name = "linear_with_residual";  // (input, weight, residual, workspace, done_counter, output)
    keep({0, 1, 2, 5});
  } else if (starts_with(n, "gang_linear") || starts_with(n, "linear_m_parallel") || n == "linear_layer" ||
             starts_with(n, "linear_cutlass_hopper")) {
    op.name = "linear";
  } else if (starts_with(n, "linear_cutlass_with_residual") || starts_with(n, "linear_swapAB_with_residual")) {
    op.name = "linear_with_residual";
  } else if (starts_with(n, "gang_attn_split_kv")) {
    op.name = "paged_attention_split_kv";  // (..., lse, output, q_workspace)
    keep({0, 1, 2, 3, 4, 5, 6, 7, 8});
  } else if (starts_with(n, "gang_attn_merge")) {
    op.name = "paged_attention_split_kv_merge";
  } else if (n == "attention" || n == "paged_attention_hopper") {
    op.name = "paged_attention";
  } else if (starts_with(n, "paged_attention_split_kv_hopper") || starts_with(n, "paged_attention_split_kv_mi300")) {
    op.name = "paged_attention_split_kv";
  } else if (starts_with(n, "splitk_linear")) {
    op.name = "splitk_linear";
  } else if (starts_with(n, "splitk_reduce")) {
    op.name = "splitk_reduce";
  }
  return op;
}

// argmax_reduce parameters beyond the reference's: [1] = first vocabulary index of this rank's LM-head shard,
// [2] != 0 = the ranks exchange their (value, index) pairs and take the global best.
int argmax_across_ranks(mk_handle* h, const RecOp& reduce, PlanOp& rd) {
  if (reduce.params.size() >= 3 && reduce.params[2] != 0) {
    if (h->cfg.world_size < 2) return 0;  // a single rank holds the whole vocabulary
    rd.flags |= mk::F_XRANK;
    rd.aux0 = (int)reduce.params[1];
    rd.note = "best (value, index) exchanged between the ranks";
  }
  return 0;
}

// A runtime-owned tensor the lowering itself needs (found by name on a re-plan).
int plan_temp_tensor(mk_handle* h, const std::string& name, int64_t rows, int64_t cols) {
  for (size_t i = 0; i < h->tensors.size(); ++i)
    if (h->tensors[i].name == name) return (int)i;
  int64_t dims[2] = {rows, cols};
  int id = add_tensor(h, name.c_str(), MK_BF16, 2, dims, nullptr);
  if (id >= 0) h->tensors[id].owned = true;
  return id;
}

int plan_graph(mk_handle* h) {
  h->plan.clear();
  h->planned = false;
  const mk_config& cfg = h->cfg;
  h->nops.clear();
  for (const RecOp& r : h->ops) h->nops.push_back(canonical_op(r));
  for (auto& t : h->tensors) {
    t.readers = 0;
    t.interleave = 0;
  }
  // operand positions that are read (everything except each layer's outputs)
  auto n_outputs = [](const RecOp& op) {
    if (starts_with(op.name, "argmax_partial")) return 2;
    if (op.name == "paged_attention_split_kv" || starts_with(op.name, "paged_attention_split_kv_sm100")) return 2;
    return 1;
  };
  for (auto& op : h->nops) {
    const int nout = n_outputs(op);
    for (int i = 0; i + nout < (int)op.t.size(); ++i)
      if (valid_tensor(h, op.t[i])) h->tensors[op.t[i]].readers++;
  }
  const bool fuse = cfg.fuse != 0;
  // RMSNorm is fused into the activation staging of the next linear; batches above 8 tokens
  // stream their activations by TMA instead, so the norm stays a task of its own there
  // Fusing the norm into the next linear makes every CTA stage (and normalise) all token
  // rows in its own shared memory: worth it for one or two tokens, beyond that the rows
  // would push the CTA past the small shared-memory carve-out and a separate rmsnorm task
  // with the linear reading activation boxes is faster.
  const bool fuse_norm = fuse && h->plan_tokens <= 2;
  // One or two tokens: linear layers run row-owner (every CTA owns whole output rows and keeps
  // the token rows resident in shared memory), provided the widest input still leaves room
  // for three weight stages inside the small carve-out.
  bool rows_mode = h->plan_tokens <= 2;
  for (const RecOp& op : h->nops) {
    if (!rows_mode || !is_linear(op.name)) continue;
    const int wi = op.name == "rmsnorm_linear" ? 2 : 1;
    if ((int)op.t.size() <= wi || !valid_tensor(h, op.t[wi]) || h->tensors[op.t[wi]].ndim != 2) continue;
    const int64_t kpad = (h->tensors[op.t[wi]].dims[1] + mk::kRowsStageK - 1) / mk::kRowsStageK * mk::kRowsStageK;
    if (h->plan_tokens * (kpad + 8) * 2 + 16 > kRowsXBudget) rows_mode = false;
  }
  h->rows_mode = rows_mode;
  // layout of fused gate/up weights: [4 gate | 4 up] per 8-row unit for the row-owner path, [64 | 64] per tile
  // otherwise; a second program over the same weights takes the primary program's layout
  const int gu_interleave = h->force_interleave ? h->force_interleave : (rows_mode ? 4 : 64);
  const int nops_all = (int)h->nops.size();
  // True when the value layer `i` writes into tensor `tid` is read by layer i+1 only:
  // walk the layers in execution order (wrapping into the next iteration) until the
  // tensor is written again.
  auto only_next_reads = [&](int i, int tid) {
    if (!h->tensors[tid].owned) return false;  // caller-visible tensors are always written
    for (int step = 1; step < nops_all; ++step) {
      const RecOp& o = h->nops[(i + step) % nops_all];
      const int nout = n_outputs(o);
      const int nin = (int)o.t.size() - nout;
      bool reads = false, writes = false;
      for (int a = 0; a < (int)o.t.size(); ++a) {
        if (o.t[a] != tid) continue;
        if (a < nin) reads = true; else writes = true;
      }
      if (reads && step != 1) return false;
      if (writes) return true;
    }
    return true;
  };
  // A norm whose output feeds the router linear right behind it AND the gate/up expert linear (the MoE layer):
  // both stage their input rows themselves, so both can apply the norm while staging.
  auto next_and_moe_w13_read = [&](int i, int tid) {
    if (!h->tensors[tid].owned) return false;
    bool seen_w13 = false;
    for (int step = 1; step < nops_all; ++step) {
      const RecOp& o = h->nops[(i + step) % nops_all];
      const int nout = n_outputs(o);
      const int nin = (int)o.t.size() - nout;
      bool reads = false, writes = false, as_input = false;
      for (int a = 0; a < (int)o.t.size(); ++a) {
        if (o.t[a] != tid) continue;
        if (a < nin) reads = true; else writes = true;
        if (a == 0) as_input = true;
      }
      if (reads) {
        const std::string& on = o.name;  // (nops hold canonical names)
        const bool w13 = (starts_with(on, "moe_w13_linear") || on == "gang_moe_w13") && as_input;
        if (step != 1 && !w13) return false;
        if (w13) seen_w13 = true;
      }
      if (writes) return seen_w13;
    }
    return seen_w13;
  };
  std::map<int, std::pair<int, int>> moe_norm;  // normalised tensor -> (its unnormalised source, the norm weight)
  int pending_route_logits = -1;                // router logits of a routing layer folded into the expert linear behind it
  int pending_norm_in = -1, pending_norm_w = -1, pending_norm_out = -1;
  const int nops = (int)h->nops.size();
  // Tensor parallelism: an allreduce layer behind a row-parallel linear is folded away.  The linear's
  // epilogue stores its fp32 sums into every rank's exchange region (F_PUSH) and the layer's output
  // tensor becomes virtual: its readers add the ranks' slots up themselves while they stage their
  // input rows (F_GATHER_IN) or fetch their residual (F_GATHER_RES).  virt maps such a tensor to the
  // ordinal of its exchange in the iteration; exchanges counts the exchanges planned so far.
  std::map<int, int> virt;
  std::map<int, int> materialised;  // virtual tensor -> exchange whose sums a stand-alone norm has stored into the tensor itself
  int exchanges = 0;
  int moe_topk = 0;  // experts per token of the latest routing layer
  // Can the output `tid` of the allreduce layer at position i stay virtual?  Every reader up to the
  // tensor's next writer must be an rmsnorm input, the input of a linear that stages its rows itself
  // (row-owner path, or the fused rmsnorm_linear layer) or a linear's residual, must come before any
  // later exchange completes, and nothing may read the tensor before position i (a value carried
  // over from the previous iteration).
  auto can_fold = [&](int i, int tid) {
    for (int j = 0; j < i; ++j) {  // a reader ahead of the tensor's first writer sees the previous iteration's value
      const RecOp& o = h->nops[j];
      const int nin = (int)o.t.size() - n_outputs(o);
      bool reads = false, writes = false;
      for (int a = 0; a < (int)o.t.size(); ++a)
        if (o.t[a] == tid) (a < nin ? reads : writes) = true;
      if (reads) return false;
      if (writes) break;
    }
    bool later_exchange = false;
    for (int j = i + 1; j < nops; ++j) {
      const RecOp& o = h->nops[j];
      const int nout = n_outputs(o);
      const int nin = (int)o.t.size() - nout;
      for (int a = 0; a < (int)o.t.size(); ++a) {
        if (o.t[a] != tid) continue;
        if (a >= nin) return o.name != "splitk_linear";  // overwritten: no more readers of this value (a split-k linear adds in place: it reads)
        if (later_exchange) return false;
        const bool lin = is_linear(o.name);
        const bool as_norm_in = (o.name == "rmsnorm" || o.name == "rmsnorm_hopper") && a == 0;
        const bool as_lin_in = lin && a == 0 && (rows_mode || o.name == "rmsnorm_linear");
        const bool as_res = lin && a == 2 && o.name.find("with_residual") != std::string::npos;
        if (!(as_norm_in || as_lin_in || as_res)) return false;
      }
      if (o.name == "allreduce") later_exchange = true;
    }
    return true;
  };
  for (int i = 0; i < nops; ++i) {
    const RecOp& op = h->nops[i];
    const std::string& nm = op.name;
    for (int id : op.t)
      if (!valid_tensor(h, id)) return h->fail(MK_E_INVALID, "layer %d (%s): bad tensor id %d", i, nm.c_str(), id);
    PlanOp po;
    if (nm == "embedding") {
      if (op.t.size() != 3) return h->fail(MK_E_INVALID, "embedding takes (input, weight, output)");
      const Tensor &ids = h->tensors[op.t[0]], &w = h->tensors[op.t[1]], &out = h->tensors[op.t[2]];
      if (ids.dtype != MK_I64) return h->fail(MK_E_INVALID, "embedding: token ids must be int64");
      if (int e = check_2d_bf16(h, op.t[1], "embedding")) return e;
      if (int e = check_2d_bf16(h, op.t[2], "embedding")) return e;
      if (w.dims[1] != out.dims[1] || w.dims[1] % 8) return h->fail(MK_E_INVALID, "embedding: hidden size mismatch");
      po.type = mk::OP_EMBED;
      po.in = op.t[0]; po.w = op.t[1]; po.out = op.t[2];
      po.n = (int)w.dims[1];
      po.aux0 = (int)w.dims[0];
    } else if (nm == "rmsnorm" || nm == "rmsnorm_hopper") {
      if (op.t.size() != 3) return h->fail(MK_E_INVALID, "rmsnorm takes (input, weight, output)");
      if (int e = check_2d_bf16(h, op.t[0], "rmsnorm")) return e;
      if (int e = check_2d_bf16(h, op.t[2], "rmsnorm")) return e;
      const Tensor &in = h->tensors[op.t[0]], &w = h->tensors[op.t[1]], &out = h->tensors[op.t[2]];
      if (w.numel() != in.dims[1] || out.dims[1] != in.dims[1] || in.dims[1] % 8)
        return h->fail(MK_E_INVALID, "rmsnorm: shape mismatch on %s", in.name.c_str());
      // fuse into the next linear when the normalised rows are only an intermediate
      if (fuse_norm && i + 1 < nops && is_linear(h->nops[i + 1].name) && h->nops[i + 1].name != "rmsnorm_linear" &&
          h->nops[i + 1].t[0] == op.t[2] && only_next_reads(i, op.t[2])) {
        pending_norm_in = op.t[0];
        pending_norm_w = op.t[1];
        pending_norm_out = op.t[2];
        continue;
      }
      if (fuse_norm && rows_mode && i + 1 < nops && is_linear(h->nops[i + 1].name) && h->nops[i + 1].name != "rmsnorm_linear" &&
          h->nops[i + 1].t[0] == op.t[2] && next_and_moe_w13_read(i, op.t[2])) {
        pending_norm_in = op.t[0];
        pending_norm_w = op.t[1];
        pending_norm_out = op.t[2];
        moe_norm[op.t[2]] = std::make_pair(op.t[0], op.t[1]);
        continue;
      }
      po.type = mk::OP_RMSNORM;
      po.in = op.t[0]; po.w = op.t[1]; po.out = op.t[2];
      po.n = (int)in.dims[1];
      if (virt.count(po.in)) {
        if (virt[po.in] != exchanges) return h->fail(MK_E_STATE, "internal: rmsnorm reads a stale exchange");
        po.flags |= mk::F_GATHER_IN;
        po.note = "input gathered from the ranks";
        // The stand-alone norm also stores the sums it gathers into the tensor's own rows (one CTA per row), so
        // that a later residual reads them with plain 16-byte loads behind the barriers in between, instead of
        // adding the ranks' words up again element by element.  (Rows of at most 8192 columns: the kernel's
        // register path.)
        if (po.n <= 8192 && h->tensors[po.in].owned) {
          po.aux0 = 1;
          materialised[po.in] = exchanges;
          po.note += ", sums stored";
        }
      }
    } else if (is_linear(nm)) {
      const bool rl = nm == "rmsnorm_linear";
      const bool sk = nm == "splitk_linear";                   // (input, weight, output)
      const bool sml = nm == "silu_mul_linear_with_residual";  // (input [gate | up], weight, residual, output)
      const bool lsilu = nm == "linear_silu";                  // (input, weight [gate/up shuffle], output = SiLU(gate) * up)
      bool with_res = nm.find("with_residual") != std::string::npos;
      const size_t want = rl ? 4 : (with_res ? 4 : 3);
      if (op.t.size() != want) return h->fail(MK_E_INVALID, "%s: expected %zu tensors", nm.c_str(), want);
      int in = op.t[0], w = rl ? op.t[2] : op.t[1], res = with_res ? op.t[2] : -1, out = op.t.back();
      if (int e = check_2d_bf16(h, in, nm.c_str())) return e;
      if (int e = check_2d_bf16(h, w, nm.c_str())) return e;
      if (int e = check_2d_bf16(h, out, nm.c_str())) return e;
      if (sk) {
        // The reference's split-K linear comes in two forms.  On sm_100 every k-split adds its
        // partial product into `output`, which already holds the residual stream
        // (tma_reduce_add in tasks/blackwell/linear_sm100_mpk.cuh:674; the model builder passes
        // output = x, python/mirage/mpk/models/qwen3/builder.py:556-563): output += input * W^T.
        // On MI300 the k-splits land in a workspace that a splitk_reduce layer sums together
        // with the residual (builder.py:537-553).  Both are one linear-with-residual task here.
        with_res = true;
        if (i + 1 < nops && h->nops[i + 1].name == "splitk_reduce" && h->nops[i + 1].t.size() == 3 &&
            h->nops[i + 1].t[0] == out) {
          res = h->nops[i + 1].t[1];
          out = h->nops[i + 1].t[2];
          if (int e = check_2d_bf16(h, out, nm.c_str())) return e;
          po.note = "split-k workspace + reduce folded";
          ++i;
        } else {
          res = out;
          po.note = "accumulates into its output";
        }
      }
      if (sml) {
        // silu_mul + linear_with_residual in one layer; the input row is [gate | up] halves
        // (tasks/ampere/silu_mul_linear.cuh:50-52).  The activation goes through a runtime-owned
        // intermediate: written by the producing gate/up linear's epilogue when that is possible,
        // else by a silu_mul task.
        const int64_t inter = h->tensors[w].dims[1];
        if (h->tensors[in].dims[1] != 2 * inter)
          return h->fail(MK_E_INVALID, "%s: input must be [gate | up] of twice the weight's K", nm.c_str());
        const int tmp = plan_temp_tensor(h, "__silu_mul_out_" + std::to_string((long long)inter), h->tensors[in].dims[0], inter);
        if (tmp < 0) return tmp;
        bool fused_up = false;
        if (fuse && i > 0 && !h->plan.empty() && is_linear(h->nops[i - 1].name) && h->nops[i - 1].t.back() == in &&
            only_next_reads(i - 1, in)) {
          PlanOp& prev = h->plan.back();
          const Tensor& pw = h->tensors[prev.w];
          if (prev.type == mk::OP_LINEAR && prev.out == in && !(prev.flags & (mk::F_RESIDUAL | mk::F_SILU_MUL | mk::F_ARGMAX)) &&
              pw.src.size() == 2 && pw.owned && pw.groups == 1 && inter % 64 == 0) {
            prev.flags |= mk::F_SILU_MUL;
            prev.out = tmp;
            prev.note += prev.note.empty() ? "silu_mul fused" : ", silu_mul fused";
            h->tensors[prev.w].interleave = gu_interleave;
            if (gu_interleave == 4 && !rows_mode) prev.flags |= mk::F_SILU4;
            fused_up = true;
          }
        }
        if (!fused_up) {
          if (inter % 8) return h->fail(MK_E_INVALID, "%s: K must be a multiple of 8", nm.c_str());
          PlanOp sm;
          sm.type = mk::OP_SILU_MUL;
          sm.in = in; sm.out = tmp;
          sm.n = (int)inter;
          sm.aux0 = (int)inter;
          sm.note = "from silu_mul_linear_with_residual";
          h->plan.push_back(sm);
        }
        in = tmp;
      }
      const Tensor &tw = h->tensors[w], &tin = h->tensors[in], &tout = h->tensors[out];
      if (tw.dims[1] != tin.dims[1]) return h->fail(MK_E_INVALID, "%s: K mismatch (%s vs %s)", nm.c_str(), tw.name.c_str(), tin.name.c_str());
      if (tw.dims[0] != (lsilu ? 2 : 1) * tout.dims[1]) return h->fail(MK_E_INVALID, "%s: N mismatch (%s vs %s)", nm.c_str(), tw.name.c_str(), tout.name.c_str());
      if (tw.dims[1] % 8 || tw.strides[0] % 8) return h->fail(MK_E_INVALID, "%s: K and the weight pitch must be multiples of 8", nm.c_str());
      if (lsilu) {
        if (!(tw.src.size() == 2 && tw.owned) || tout.dims[1] % 64)
          return h->fail(MK_E_UNSUPPORTED, "%s: the weight must come from shuffle_tensors([gate, up]) and the output width be a multiple of 64", nm.c_str());
        po.flags |= mk::F_SILU_MUL;
        po.note = "silu_mul fused";
        h->tensors[w].interleave = gu_interleave;
        if (gu_interleave == 4 && !rows_mode) po.flags |= mk::F_SILU4;
      }
      po.type = mk::OP_LINEAR;
      if (rows_mode) po.flags |= mk::F_ROWS;
      po.in = in; po.w = w; po.out = out; po.res = res;
      po.n = (int)tw.dims[0];
      po.k = (int)tw.dims[1];
      if (with_res) {
        if (int e = check_2d_bf16(h, res, nm.c_str())) return e;
        po.flags |= mk::F_RESIDUAL;
        if (cfg.world_size > 1) po.flags |= mk::F_RES_RANK0;  // row-parallel partial sums: add the residual once
      }
      if (rl) {
        po.flags |= mk::F_NORM_IN;
        po.norm_w = op.t[1];
      } else if (pending_norm_out == in) {
        po.flags |= mk::F_NORM_IN;
        po.norm_w = pending_norm_w;
        po.in = pending_norm_in;
        po.note += po.note.empty() ? "rmsnorm fused" : ", rmsnorm fused";
      }
      pending_norm_in = pending_norm_w = pending_norm_out = -1;
      if (virt.count(po.in)) {
        if (virt[po.in] != exchanges) return h->fail(MK_E_STATE, "internal: a linear reads a stale exchange");
        po.flags |= mk::F_GATHER_IN;
        po.note += po.note.empty() ? "input gathered from the ranks" : ", input gathered from the ranks";
      }
      if (po.res >= 0 && virt.count(po.res)) {
        if (virt[po.res] != exchanges) return h->fail(MK_E_STATE, "internal: a residual reads a stale exchange");
        if (materialised.count(po.res) && materialised[po.res] == exchanges) {
          po.note += po.note.empty() ? "residual: the sums a norm stored" : ", residual: the sums a norm stored";
        } else {
          po.flags |= mk::F_GATHER_RES;
          po.note += po.note.empty() ? "residual gathered from the ranks" : ", residual gathered from the ranks";
        }
      }
      // SiLU*up fused into the epilogue of a gate/up linear
      if (fuse && !with_res && !(po.flags & mk::F_SILU_MUL) && i + 1 < nops && h->nops[i + 1].name == "silu_mul" && h->nops[i + 1].t.size() == 2 &&
          h->nops[i + 1].t[0] == out && only_next_reads(i, out) && tw.src.size() == 2 && tw.owned) {
        const RecOp& sm = h->nops[i + 1];
        const Tensor& so = h->tensors[sm.t[1]];
        const int64_t inter = so.dims[1];
        const int64_t blk = inter / std::max(1, sm.grid[0]);
        const Tensor &g = h->tensors[tw.src[0]], &u = h->tensors[tw.src[1]];
        if (g.dims[0] == inter && u.dims[0] == inter && inter % 64 == 0 && tw.groups > 0 && inter / tw.groups == blk &&
            inter % std::max(1, sm.grid[0]) == 0) {
          po.flags |= mk::F_SILU_MUL;
          po.out = sm.t[1];
          po.note += po.note.empty() ? "silu_mul fused" : ", silu_mul fused";
          h->tensors[w].interleave = gu_interleave;
        if (gu_interleave == 4 && !rows_mode) po.flags |= mk::F_SILU4;
          ++i;
        }
      }
      // per-tile argmax partials fused into the LM-head epilogue
      if (fuse && !(po.flags & mk::F_SILU_MUL) && i + 2 < nops && starts_with(h->nops[i + 1].name, "argmax_partial") &&
          starts_with(h->nops[i + 2].name, "argmax_reduce") && h->nops[i + 1].t[0] == out) {
        po.flags |= mk::F_ARGMAX;
        po.amax_n = (po.n + mk::kTileRows - 1) / mk::kTileRows;
        po.note += po.note.empty() ? "argmax partials fused" : ", argmax partials fused";
        h->plan.push_back(po);
        PlanOp rd;
        rd.type = mk::OP_ARGMAX_REDUCE;
        rd.flags = 0;  // CTA 0 alone up to 8 tokens, the whole grid beyond (decided on the device)
        rd.out = h->nops[i + 2].t.back();
        rd.amax_n = po.amax_n;
        rd.in = -2;  // reads the previous op's partials
        if (int e = argmax_across_ranks(h, h->nops[i + 2], rd)) return e;
        if (h->tensors[rd.out].dtype != MK_I64) return h->fail(MK_E_INVALID, "argmax output must be int64");
        h->plan.push_back(rd);
        i += 2;
        continue;
      }
    } else if (nm == "paged_attention" || starts_with(nm, "paged_attention_sm100") ||
               nm == "paged_attention_split_kv" || starts_with(nm, "paged_attention_split_kv_sm100")) {
      const bool split = nm.find("split_kv") != std::string::npos;
      if (op.t.size() != (split ? 9u : 8u)) return h->fail(MK_E_INVALID, "%s: wrong operand count", nm.c_str());
      int out = op.t[7];
      if (split) {
        if (i + 1 >= nops || !starts_with(h->nops[i + 1].name, "paged_attention_split_kv_merge"))
          return h->fail(MK_E_UNSUPPORTED, "paged_attention_split_kv must be followed by its merge layer");
        const RecOp& mg = h->nops[i + 1];
        if (mg.t.size() != 3) return h->fail(MK_E_INVALID, "split_kv merge takes (lse, output_tmp, output)");
        out = mg.t[2];
      }
      if (op.params.size() < 4) return h->fail(MK_E_INVALID, "%s: params (q heads, kv heads, qk_norm, rope) missing", nm.c_str());
      po.type = mk::OP_ATTN;
      po.in = op.t[0]; po.kc = op.t[1]; po.vc = op.t[2]; po.qn = op.t[3]; po.kn = op.t[4];
      po.cos = op.t[5]; po.sin = op.t[6]; po.out = out;
      po.aux1 = (int)op.params[0];
      po.aux0 = (int)op.params[1];
      if (op.params[2]) po.flags |= mk::F_QK_NORM;
      if (op.params[3]) po.flags |= mk::F_ROPE;
      const Tensor &kc = h->tensors[po.kc], &qkv = h->tensors[po.in], &to = h->tensors[out];
      if (kc.ndim != 4 || kc.dims[3] != mk::kHeadDim) return h->fail(MK_E_UNSUPPORTED, "attention: head_dim must be 128");
      if (kc.dims[0] != cfg.max_num_pages || kc.dims[1] != cfg.page_size || kc.dims[2] != po.aux0)
        return h->fail(MK_E_INVALID, "attention: KV cache must be [max_num_pages, page_size, kv_heads, 128]");
      const int qpk = po.aux0 > 0 ? po.aux1 / po.aux0 : 0;
      if (po.aux0 <= 0 || po.aux1 % po.aux0 || (qpk != 1 && qpk != 2 && qpk != 4 && qpk != 8))
        return h->fail(MK_E_UNSUPPORTED, "attention: q heads per kv head must be 1, 2, 4 or 8");
      if (qkv.dims[1] != (int64_t)(po.aux1 + 2 * po.aux0) * mk::kHeadDim || to.dims[1] != (int64_t)po.aux1 * mk::kHeadDim)
        return h->fail(MK_E_INVALID, "attention: qkv/output widths do not match the head counts");
      po.aux2 = (int)h->tensors[po.cos].dims[0];
      if (split) { po.note = "split-kv + merge"; ++i; }
    } else if (nm == "splitk_reduce") {
      return h->fail(MK_E_UNSUPPORTED, "splitk_reduce without a preceding splitk_linear that writes its workspace");
    } else if (starts_with(nm, "paged_attention_split_kv_merge")) {
      return h->fail(MK_E_UNSUPPORTED, "split_kv merge without a preceding split_kv layer");
    } else if (nm == "silu_mul") {
      if (op.t.size() != 2) return h->fail(MK_E_INVALID, "silu_mul takes (input, output)");
      if (int e = check_2d_bf16(h, op.t[0], "silu_mul")) return e;
      if (int e = check_2d_bf16(h, op.t[1], "silu_mul")) return e;
      const Tensor &in = h->tensors[op.t[0]], &out = h->tensors[op.t[1]];
      const int64_t blk = out.dims[1] / std::max(1, op.grid[0]);
      if (in.dims[1] != 2 * out.dims[1] || blk * op.grid[0] != out.dims[1] || blk % 8)
        return h->fail(MK_E_INVALID, "silu_mul: input must be [gate|up] blocks of a multiple of 8 columns");
      po.type = mk::OP_SILU_MUL;
      po.in = op.t[0]; po.out = op.t[1];
      po.n = (int)out.dims[1];
      po.aux0 = (int)blk;
    } else if (starts_with(nm, "argmax_partial") || nm == "argmax") {
      const bool single = nm == "argmax";
      if (!single && (i + 1 >= nops || !starts_with(h->nops[i + 1].name, "argmax_reduce")))
        return h->fail(MK_E_UNSUPPORTED, "argmax_partial must be followed by argmax_reduce");
      if (int e = check_2d_bf16(h, op.t[0], "argmax")) return e;
      const int out = single ? op.t[1] : h->nops[i + 1].t.back();
      if (h->tensors[out].dtype != MK_I64) return h->fail(MK_E_INVALID, "argmax output must be int64");
      po.type = mk::OP_ARGMAX_PARTIAL;
      po.in = op.t[0];
      po.n = (int)h->tensors[op.t[0]].dims[1];
      po.amax_n = std::max(1, std::min(po.n / 256, 1024));
      h->plan.push_back(po);
      PlanOp rd;
      rd.type = mk::OP_ARGMAX_REDUCE;
      rd.flags = 0;  // CTA 0 alone up to 8 tokens, the whole grid beyond (decided on the device)
      rd.out = out;
      rd.amax_n = po.amax_n;
      rd.in = -2;
      if (!single)
        if (int e = argmax_across_ranks(h, h->nops[i + 1], rd)) return e;
      h->plan.push_back(rd);
      if (!single) ++i;
      continue;
    } else if (starts_with(nm, "argmax_reduce")) {
      return h->fail(MK_E_UNSUPPORTED, "argmax_reduce without a preceding argmax_partial");
    } else if (nm == "allreduce") {
      if (op.t.size() != 3) return h->fail(MK_E_INVALID, "allreduce takes (input, buffer, output)");
      if (int e = check_2d_bf16(h, op.t[0], "allreduce")) return e;
      if (int e = check_2d_bf16(h, op.t[2], "allreduce")) return e;
      const Tensor &in = h->tensors[op.t[0]], &out = h->tensors[op.t[2]];
      if (in.dims[1] != out.dims[1] || in.dims[1] % 8) return h->fail(MK_E_INVALID, "allreduce: column counts must match and be a multiple of 8");
      if (op.params.size() >= 2 && (op.params[0] != cfg.world_size || op.params[1] != cfg.rank))
        return h->fail(MK_E_INVALID, "allreduce: (num_gpus, my_gpu_id) differ from the constructor's world_size / mpi_rank");
      if (cfg.world_size > 8) return h->fail(MK_E_UNSUPPORTED, "at most 8 ranks");
      exchanges += 1;
      if (fuse && cfg.world_size > 1 && i > 0 && !h->plan.empty()) {
        PlanOp& prev = h->plan.back();
        if (prev.type == mk::OP_LINEAR && prev.out == op.t[0] && !(prev.flags & (mk::F_SILU_MUL | mk::F_ARGMAX)) &&
            is_linear(h->nops[i - 1].name) && h->tensors[op.t[0]].owned && h->tensors[op.t[2]].owned &&
            only_next_reads(i - 1, op.t[0]) && can_fold(i, op.t[2])) {
          prev.flags |= mk::F_PUSH;
          prev.note += prev.note.empty() ? "allreduce folded: sums pushed to all ranks" : ", allreduce folded: sums pushed to all ranks";
          virt[op.t[2]] = exchanges;
          continue;
        }
      }
      virt.erase(op.t[2]);
      po.type = mk::OP_ALLREDUCE;
      po.in = op.t[0]; po.out = op.t[2];  // the reference's staging buffer (operand 1) is replaced by the exchange region
      po.n = (int)in.dims[1];
      po.aux0 = cfg.world_size;
      po.aux1 = cfg.rank;
    } else if (nm == "tensor_init") {
      continue;  // the reference zeroes an accumulation buffer here; nothing accumulates in place in this runtime
    } else if (starts_with(nm, "moe_topk_softmax")) {
      // (router logits [T, experts]) -> (top-k weights [T, k], routing indices, mask): the reference's index
      // and mask tensors describe ITS grouping of tokens per expert; this runtime keeps its own [T, k] tables
      if (op.t.size() != 4) return h->fail(MK_E_INVALID, "moe_topk_softmax takes (input, topk_weight, routing_indices, mask)");
      if (int e = check_2d_bf16(h, op.t[0], nm.c_str())) return e;
      const Tensor &in = h->tensors[op.t[0]], &tw = h->tensors[op.t[1]];
      if (tw.ndim != 2 || tw.dims[1] < 1 || tw.dims[1] > 32 || in.dims[1] > 256 || tw.dims[1] > in.dims[1])
        return h->fail(MK_E_UNSUPPORTED, "moe routing: at most 256 experts and 32 experts per token");
      moe_topk = (int)tw.dims[1];
      // routing right in front of the gate/up expert linear: that op routes the tokens itself (no op, no barrier)
      if (fuse && rows_mode && i + 1 < nops &&
          (starts_with(h->nops[i + 1].name, "moe_w13_linear") || h->nops[i + 1].name == "gang_moe_w13")) {
        pending_route_logits = op.t[0];
        continue;
      }
      po.type = mk::OP_MOE_ROUTE;
      po.in = op.t[0];
      po.out = op.t[1];
      po.aux0 = (int)tw.dims[1];
      po.aux1 = (int)in.dims[1];
    } else if (starts_with(nm, "moe_w13_linear") || starts_with(nm, "moe_w2_linear") || starts_with(nm, "gang_moe_w")) {
      // (input, weight [experts, n, K], routing_indices, mask, output [T, k, n])
      if (op.t.size() != 5) return h->fail(MK_E_INVALID, "%s takes (input, weight, routing_indices, mask, output)", nm.c_str());
      if (!rows_mode) return h->fail(MK_E_UNSUPPORTED, "mixture-of-experts layers are built for one or two batched tokens (every (token, expert) pair a row-owner GEMV); a grouped GEMM for wider batches is not");
      if (moe_topk <= 0) return h->fail(MK_E_INVALID, "%s: no moe_topk_softmax_routing layer before it", nm.c_str());
      const bool w2 = nm.find("w2") != std::string::npos;
      const Tensor &in = h->tensors[op.t[0]], &w = h->tensors[op.t[1]], &out = h->tensors[op.t[4]];
      if (w.ndim != 3 || w.dtype != MK_BF16 || in.dtype != MK_BF16 || out.dtype != MK_BF16)
        return h->fail(MK_E_INVALID, "%s: the weight must be [experts, n, K] bf16", nm.c_str());
      if (w.strides[2] != 1 || w.strides[1] != w.dims[2] || w.strides[0] != w.dims[1] * w.dims[2])
        return h->fail(MK_E_INVALID, "%s: the weight must be contiguous", nm.c_str());
      const int64_t K = w.dims[2], N = w.dims[1];
      if (in.dims[in.ndim - 1] != K || out.dims[out.ndim - 1] != N || N % 8 || K % 8)
        return h->fail(MK_E_INVALID, "%s: input / output widths do not match the weight", nm.c_str());
      if ((w2 && in.ndim != 3) || (!w2 && in.ndim != 2) || out.ndim != 3 || out.dims[1] != moe_topk)
        return h->fail(MK_E_INVALID, "%s: input must be [T, K]%s and output [T, k, n]", nm.c_str(), w2 ? " per (token, slot) pair, i.e. [T, k, K]" : "");
      po.type = mk::OP_MOE_LINEAR;
      po.flags |= mk::F_ROWS | (w2 ? mk::F_MOE_PAIR_IN : 0);
      po.in = op.t[0]; po.w = op.t[1]; po.out = op.t[4];
      if (!w2 && pending_route_logits >= 0) {
        po.res = pending_route_logits;
        po.flags |= mk::F_MOE_ROUTE;
        po.note += po.note.empty() ? "routing folded in" : ", routing folded in";
        pending_route_logits = -1;
      }
      if (!w2 && moe_norm.count(op.t[0])) {  // the norm in front of the layer is applied while the rows are staged
        po.in = moe_norm[op.t[0]].first;
        po.norm_w = moe_norm[op.t[0]].second;
        po.flags |= mk::F_NORM_IN;
        po.note += po.note.empty() ? "rmsnorm fused" : ", rmsnorm fused";
      }
      po.n = (int)N;
      po.k = (int)K;
      po.aux0 = moe_topk;
      po.aux1 = (int)w.dims[0];
    } else if (nm == "moe_silu_mul") {
      // [T, k, 2 * inter] in [gate | up] halves -> [T, k, inter]: the dense silu_mul op over T * k rows
      if (op.t.size() != 2) return h->fail(MK_E_INVALID, "moe_silu_mul takes (input, output)");
      const Tensor &in = h->tensors[op.t[0]], &out = h->tensors[op.t[1]];
      if (in.ndim != 3 || out.ndim != 3 || in.dims[2] != 2 * out.dims[2] || out.dims[2] % 8 || in.dtype != MK_BF16)
        return h->fail(MK_E_INVALID, "moe_silu_mul: input [T, k, 2 * inter], output [T, k, inter], bf16");
      po.type = mk::OP_SILU_MUL;
      po.in = op.t[0]; po.out = op.t[1];
      po.n = (int)out.dims[2];
      po.aux0 = (int)out.dims[2];
      po.aux1 = (int)out.dims[1];  // rows per token
    } else if (starts_with(nm, "moe_mul_sum_add")) {
      // (input [T, k, n], weight [T, k], residual [T, n], output [T, n])
      if (op.t.size() != 4) return h->fail(MK_E_INVALID, "moe_mul_sum_add takes (input, weight, residual, output)");
      const Tensor &in = h->tensors[op.t[0]], &out = h->tensors[op.t[3]];
      if (in.ndim != 3 || out.ndim != 2 || in.dims[2] != out.dims[1] || out.dims[1] % 8)
        return h->fail(MK_E_INVALID, "moe_mul_sum_add: input [T, k, n], output [T, n]");
      if (int e = check_2d_bf16(h, op.t[2], nm.c_str())) return e;
      // right behind the down projection of the experts, and its only reader: that op adds the slots up itself
      if (fuse && rows_mode && !h->plan.empty() && in.dims[1] <= 8) {
        PlanOp& prev = h->plan.back();
        if (prev.type == mk::OP_MOE_LINEAR && (prev.flags & mk::F_MOE_PAIR_IN) && prev.out == op.t[0] && h->tensors[op.t[0]].owned &&
            only_next_reads(i - 1, op.t[0]) && canonical_name_is_w2(h->nops[i - 1].name)) {
          prev.flags |= mk::F_MOE_COMBINE;
          prev.res = op.t[2];
          prev.out = op.t[3];
          prev.note += prev.note.empty() ? "weighted sum folded in" : ", weighted sum folded in";
          continue;
        }
      }
      po.type = mk::OP_MOE_COMBINE;
      po.in = op.t[0]; po.res = op.t[2]; po.out = op.t[3];
      po.n = (int)out.dims[1];
      po.aux0 = (int)in.dims[1];
    } else {
      return h->fail(MK_E_UNSUPPORTED, "unknown layer '%s'", nm.c_str());
    }
    if (pending_norm_out >= 0 && po.type != 0) {
      return h->fail(MK_E_STATE, "internal: a fused rmsnorm lost its linear");
    }
    h->plan.push_back(po);
  }
  // every op waits for its producers; CTA-0-only ops that follow each other need no grid barrier
  for (size_t i = 0; i < h->plan.size(); ++i) h->plan[i].flags |= mk::F_SYNC_BEFORE;
  if (h->plan.empty()) return h->fail(MK_E_INVALID, "no layers recorded");
  // the first op follows the iteration's own barrier (offline) or the launch (onepass)
  h->plan[0].flags &= ~mk::F_SYNC_BEFORE;
  // An op whose only dependency on its predecessor is a gathered input needs no grid barrier: every
  // exchange word says by itself whether it has arrived.  (The op must not write what the pushing
  // linear before it still reads.)
  for (size_t i = 1; i < h->plan.size(); ++i) {
    PlanOp& cur = h->plan[i];
    const PlanOp& prev = h->plan[i - 1];
    if ((cur.flags & mk::F_GATHER_IN) && (prev.flags & mk::F_PUSH) && cur.out != prev.in && cur.out != prev.res &&
        !(cur.flags & mk::F_GATHER_RES) && cur.res < 0)
      cur.flags &= ~mk::F_SYNC_BEFORE;
  }
  h->planned = true;
  return 0;
}

const char* op_type_name(int t) {
  switch (t) {
    case mk::OP_EMBED: return "embed";
    case mk::OP_RMSNORM: return "rmsnorm";
    case mk::OP_LINEAR: return "linear";
    case mk::OP_ATTN: return "attention";
    case mk::OP_SILU_MUL: return "silu_mul";
    case mk::OP_ARGMAX_PARTIAL: return "argmax_partial";
    case mk::OP_ARGMAX_REDUCE: return "argmax_reduce";
    case mk::OP_ALLREDUCE: return "allreduce";
    case mk::OP_MOE_ROUTE: return "moe_route";
    case mk::OP_MOE_LINEAR: return "moe_linear";
    case mk::OP_MOE_COMBINE: return "moe_combine";
  }
  return "?";
}

// ------------------------------------------------------------------------------------
// device side of compile
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int materialise_shuffle(mk_handle* h, Tensor& t) {
  // rows of the sources, interleaved per group; every source is a full-row 2-D bf16 tensor
  const size_t row_bytes = (size_t)t.dims[1] * dtype_size(t.dtype);
  size_t dst_row = 0;
  auto copy_rows = [&](const Tensor& s, int64_t r0, int64_t nr) -> int {
    const char* sp = (const char*)s.ptr + (size_t)r0 * s.strides[0] * dtype_size(s.dtype);
    cudaError_t e;
    if (s.strides[0] == s.dims[1])
      e = cudaMemcpyAsync((char*)t.ptr + dst_row * row_bytes, sp, (size_t)nr * row_bytes, cudaMemcpyDeviceToDevice, 0);
    else
      e = cudaMemcpy2DAsync((char*)t.ptr + dst_row * row_bytes, row_bytes, sp, (size_t)s.strides[0] * dtype_size(s.dtype),
                            row_bytes, (size_t)nr, cudaMemcpyDeviceToDevice, 0);
    dst_row += nr;
    return e == cudaSuccess ? 0 : h->cuda_fail(e, "shuffle copy");
  };
  if (t.interleave > 0) {
    // one strided copy per source: "rows" of g weight rows each, placed 2g rows apart
    const int64_t g = t.interleave;
    for (int which = 0; which < 2; ++which) {
      const Tensor& s = h->tensors[t.src[which]];
      if (s.strides[0] != s.dims[1] || s.dims[0] % g) return h->fail(MK_E_UNSUPPORTED, "gate/up weights must be dense with a multiple of %d rows", (int)g);
      cudaError_t e = cudaMemcpy2DAsync((char*)t.ptr + (size_t)which * g * row_bytes, 2 * g * row_bytes, s.ptr, g * row_bytes,
                                        g * row_bytes, (size_t)(s.dims[0] / g), cudaMemcpyDeviceToDevice, 0);
      if (e != cudaSuccess) return h->cuda_fail(e, "gate/up interleave copy");
    }
  } else {
    for (int g = 0; g < t.groups; ++g)
      for (int sid : t.src) {
        const Tensor& s = h->tensors[sid];
        const int64_t per = s.dims[0] / t.groups;
        if (int e = copy_rows(s, g * per, per)) return e;
      }
  }
  return 0;
}

}  // namespace

// ------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------
extern "C" {

mk_handle* mk_create(const mk_config* cfg) {
  if (!cfg) return nullptr;
  mk_handle* h = new mk_handle();
  h->cfg = *cfg;
  if (h->cfg.timeout_ms <= 0) h->cfg.timeout_ms = 4000;
  if ((h->cfg.debug_flags & 15) != 0)
    fprintf(stderr, "b200mk: debug_flags=0x%x: measurement mode, the kernel skips arithmetic and its results are WRONG\n",
            h->cfg.debug_flags);
  return h;
}

int mk_last_error(mk_handle* h, char* buf, int n) {
  if (!h || !buf || n <= 0) return MK_E_INVALID;
  snprintf(buf, n, "%s", h->err.c_str());
  return 0;
}

int mk_tensor_attach(mk_handle* h, const char* name, void* ptr, int dtype, int ndim, const int64_t* dims,
                     const int64_t* strides) {
  if (!h) return MK_E_INVALID;
  if (h->planned) return h->fail(MK_E_STATE, "graph already compiled");
  if (!ptr) return h->fail(MK_E_INVALID, "attach_input %s: null pointer", name ? name : "?");
  if (((uintptr_t)ptr) & 15) return h->fail(MK_E_INVALID, "attach_input %s: pointer must be 16-byte aligned", name);
  if (strides)
    for (int d = 0; d + 1 < ndim; ++d)
      if (strides[d] != strides[d + 1] * dims[d + 1])
        return h->fail(MK_E_INVALID, "attach_input %s: tensor must be row-major contiguous", name);
  int id = add_tensor(h, name, dtype, ndim, dims, strides);
  if (id < 0) return id;
  h->tensors[id].ptr = ptr;
  h->tensors[id].user = true;
  return id;
}

int mk_tensor_new(mk_handle* h, const char* name, int dtype, int ndim, const int64_t* dims, const int64_t* strides,
                  int category) {
  if (!h) return MK_E_INVALID;
  if (h->planned) return h->fail(MK_E_STATE, "graph already compiled");
  if (category != MK_CAT_CUDA && category != MK_CAT_SYMMETRIC) return h->fail(MK_E_INVALID, "Invalid io_category");
  int id = add_tensor(h, name, dtype, ndim, dims, strides);
  if (id < 0) return id;
  h->tensors[id].owned = true;
  return id;
}

static int shuffle_impl(mk_handle* h, const char* name, const int* ids, int n, int dim, int groups) {
  if (!h) return MK_E_INVALID;
  if (h->planned) return h->fail(MK_E_STATE, "graph already compiled");
  if (dim != 0) return h->fail(MK_E_UNSUPPORTED, "only dimension 0 can be shuffled");
  if (n < 1 || groups < 1 || !ids) return h->fail(MK_E_INVALID, "shuffle_tensors: need inputs and num_groups >= 1");
  int64_t rows = 0, cols = -1;
  for (int i = 0; i < n; ++i) {
    if (!valid_tensor(h, ids[i])) return h->fail(MK_E_INVALID, "shuffle_tensors: bad tensor id");
    const Tensor& s = h->tensors[ids[i]];
    if (s.ndim != 2) return h->fail(MK_E_INVALID, "shuffle_tensors: inputs must be 2-D");
    if (cols >= 0 && s.dims[1] != cols) return h->fail(MK_E_INVALID, "shuffle_tensors: column counts differ");
    if (s.dims[0] % groups) return h->fail(MK_E_INVALID, "shuffle_tensors: rows of %s not divisible by num_groups", s.name.c_str());
    if (s.dtype != h->tensors[ids[0]].dtype) return h->fail(MK_E_INVALID, "shuffle_tensors: dtypes differ");
    cols = s.dims[1];
    rows += s.dims[0];
  }
  int64_t dims[2] = {rows, cols};
  int id = add_tensor(h, name ? name : "shuffled", h->tensors[ids[0]].dtype, 2, dims, nullptr);
  if (id < 0) return id;
  Tensor& t = h->tensors[id];
  t.owned = true;
  t.src.assign(ids, ids + n);
  t.groups = groups;
  return id;
}

int mk_tensor_shuffle(mk_handle* h, const char* name, const int* ids, int n, int dim, int groups) {
  return shuffle_impl(h, name, ids, n, dim, groups);
}
int mk_tensor_fuse(mk_handle* h, const char* name, const int* ids, int n, int dim, int groups) {
  return shuffle_impl(h, name, ids, n, dim, groups);
}

int mk_op(mk_handle* h, const char* op_name, const int* ids, int n, const int64_t* params, int np, const int* grid,
          const int* block) {
  if (!h) return MK_E_INVALID;
  if (h->planned) return h->fail(MK_E_STATE, "graph already compiled");
  if (!op_name || n < 1 || !ids) return h->fail(MK_E_INVALID, "mk_op: name and tensors required");
  RecOp op;
  op.name = op_name;
  op.t.assign(ids, ids + n);
  if (params && np > 0) op.params.assign(params, params + np);
  for (int i = 0; i < 3; ++i) {
    op.grid[i] = grid ? std::max(1, grid[i]) : 1;
    op.block[i] = block ? std::max(1, block[i]) : 1;
  }
  h->ops.push_back(op);
  return (int)h->ops.size() - 1;
}

int mk_set_meta(mk_handle* h, void* const meta[10], int64_t total_num_requests, void* profiler) {
  (void)profiler;
  if (!h || !meta) return MK_E_INVALID;
  for (int i = 0; i < 10; ++i) {
    if (!meta[i]) return h->fail(MK_E_INVALID, "meta tensor %d is null", i);
    h->meta[i] = meta[i];
  }
  if (total_num_requests < 1) return h->fail(MK_E_INVALID, "total_num_requests must be >= 1");
  h->total_requests = total_num_requests;
  h->meta_set = true;
  return 0;
}

int mk_set_profiler(mk_handle* h, void* ptr, int64_t n_entries) {
  if (!h) return MK_E_INVALID;
  if (h->compiled) return h->fail(MK_E_STATE, "set the profiler buffer before compile");
  if (ptr && (n_entries <= 0 || (((uintptr_t)ptr) & 7))) return h->fail(MK_E_INVALID, "profiler buffer must be 8-byte aligned and non-empty");
  h->prof_ptr = ptr;
  h->prof_entries = ptr ? n_entries : 0;
  return 0;
}

// Size of this rank's exchange region for the allreduce layers of the planned graph (0 if none).
static size_t xchg_bytes(mk_handle* h) {
  int cols = 0;
  bool amax = false;
  auto scan = [&](const std::vector<PlanOp>& plan) {
    for (const PlanOp& po : plan) {
      if (po.type == mk::OP_ALLREDUCE || (po.type == mk::OP_LINEAR && (po.flags & mk::F_PUSH))) cols = std::max(cols, po.n);
      if (po.type == mk::OP_ARGMAX_REDUCE && (po.flags & mk::F_XRANK)) amax = true;
    }
  };
  scan(h->plan);
  for (int i = 0; i < h->nprog; ++i) scan(h->prog[i].plan);
  if ((cols == 0 && !amax) || h->cfg.world_size < 2) return 0;
  h->xchg_tokens = h->cfg.max_num_batched_tokens;
  h->xchg_cols = std::max(cols, 8);
  // two halves x ranks x token rows x columns of 8-byte {value, exchange number} words, then the argmax area
  h->xchg_amax_word = (long long)2 * h->cfg.world_size * h->xchg_tokens * h->xchg_cols;
  return ((size_t)h->xchg_amax_word + (size_t)h->cfg.world_size * h->xchg_tokens * 2) * 8;
}

int mk_comm_prepare(mk_handle* h, unsigned char handle_out[64]) {
  if (!h || !handle_out) return MK_E_INVALID;
  if (h->compiled) return h->fail(MK_E_STATE, "already compiled");
  if (int e = mk_plan(h)) return e;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memset(handle_out, 0, 64);
  const size_t bytes = xchg_bytes(h);
  if (bytes == 0) return 0;  // nothing to exchange (single rank or no allreduce layer)
  if (!h->xchg_local)
    if (int e = h->dmalloc(&h->xchg_local, bytes)) return e;
  cudaIpcMemHandle_t ipc;
  cudaError_t ce = cudaIpcGetMemHandle(&ipc, h->xchg_local);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "cudaIpcGetMemHandle");
  memcpy(handle_out, &ipc, 64);
  return 1;
}

int mk_comm_connect(mk_handle* h, const unsigned char* handles, int n) {
  if (!h || !handles) return MK_E_INVALID;
  if (n != h->cfg.world_size) return h->fail(MK_E_INVALID, "expected %d handles, got %d", h->cfg.world_size, n);
  if (!h->xchg_local) return h->fail(MK_E_STATE, "mk_comm_prepare must come first");
  for (int r = 0; r < n; ++r) {
    if (r == h->cfg.rank) {
      h->xchg_peer[r] = h->xchg_local;
      continue;
    }
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, handles + (size_t)r * 64, 64);
    cudaError_t ce = cudaIpcOpenMemHandle(&h->xchg_peer[r], ipc, cudaIpcMemLazyEnablePeerAccess);
    if (ce != cudaSuccess) return h->cuda_fail(ce, "cudaIpcOpenMemHandle (is the peer GPU reachable over NVLink/PCIe?)");
  }
  h->xchg_ready = true;
  return 0;
}

// Shape class of an iteration width: which path and activation-box height the linears get.
static int width_class(int tokens) { return tokens <= 2 ? 2 : (tokens <= 8 ? 8 : (tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64))); }
// Two programs when prompt chunks make some iterations wider than the decode iterations can be and the
// two widths put the linears on different paths (otherwise one program planned for the wider one serves all).
static bool two_programs(const mk_config& c) {
  return c.mode == MK_MODE_OFFLINE && c.max_num_batched_tokens > c.max_num_batched_requests &&
         width_class(c.max_num_batched_tokens) != width_class(c.max_num_batched_requests);
}

int mk_plan(mk_handle* h) {
  if (!h) return MK_E_INVALID;
  const mk_config& c = h->cfg;
  if (c.mode != MK_MODE_OFFLINE && c.mode != MK_MODE_ONEPASS) return h->fail(MK_E_INVALID, "Invalid persistent kernel mode");
  if (c.max_num_batched_requests < 1 || c.max_num_batched_tokens < c.max_num_batched_requests)
    return h->fail(MK_E_INVALID, "max_num_batched_tokens must be >= max_num_batched_requests >= 1");
  if (c.max_num_batched_tokens > 128) return h->fail(MK_E_UNSUPPORTED, "at most 128 batched tokens");
  if (c.page_size < 1 || c.max_num_pages < 1 || c.max_seq_length < 2) return h->fail(MK_E_INVALID, "bad paging/sequence limits");
  if (c.page_size & (c.page_size - 1)) return h->fail(MK_E_UNSUPPORTED, "page_size must be a power of two (got %d)", c.page_size);
  if (c.world_size < 1 || c.rank < 0 || c.rank >= c.world_size) return h->fail(MK_E_INVALID, "bad rank/world_size");
  h->force_interleave = 0;
  h->plan_tokens = two_programs(c) ? c.max_num_batched_requests : c.max_num_batched_tokens;
  return plan_graph(h);
}

int mk_num_device_ops(mk_handle* h) { return h && h->planned ? (int)h->plan.size() : MK_E_STATE; }

int mk_describe(mk_handle* h, char* buf, int n) {
  if (!h || !buf || n <= 0) return MK_E_INVALID;
  if (!h->planned) return h->fail(MK_E_STATE, "not planned");
  std::string s;
  char line[512];
  for (size_t i = 0; i < h->plan.size(); ++i) {
    const PlanOp& p = h->plan[i];
    snprintf(line, sizeof(line), "%zu %s n=%d k=%d flags=0x%x in=%s out=%s%s%s\n", i, op_type_name(p.type), p.n, p.k,
             p.flags, p.in >= 0 ? h->tensors[p.in].name.c_str() : "-", p.out >= 0 ? h->tensors[p.out].name.c_str() : "-",
             p.note.empty() ? "" : " # ", p.note.c_str());
    s += line;
  }
  snprintf(buf, n, "%s", s.c_str());
  return (int)h->plan.size();
}

int mk_grid_size(mk_handle* h) { return h && h->compiled ? h->grid : MK_E_STATE; }
int64_t mk_weight_bytes_per_step(mk_handle* h) { return h && h->compiled ? h->weight_bytes : MK_E_STATE; }

void* mk_tensor_ptr(mk_handle* h, int id) {
  if (!h || !valid_tensor(h, id)) return nullptr;
  return h->tensors[id].ptr;
}

int mk_tensor_read(mk_handle* h, int id, void* host_buf, int64_t bytes) {
  if (!h || !host_buf || !valid_tensor(h, id)) return MK_E_INVALID;
  const Tensor& t = h->tensors[id];
  if (!t.ptr) return h->fail(MK_E_STATE, "tensor %s has no storage before compile", t.name.c_str());
  if (bytes < 0 || (size_t)bytes > t.alloc_bytes()) return h->fail(MK_E_INVALID, "tensor %s holds %zu bytes", t.name.c_str(), t.alloc_bytes());
  cudaError_t ce = cudaMemcpy(host_buf, t.ptr, (size_t)bytes, cudaMemcpyDeviceToHost);
  return ce == cudaSuccess ? 0 : h->cuda_fail(ce, "tensor readback");
}

int mk_debug_partition(int64_t nblk, int64_t nkt, int grid, int64_t* begin_out, int* owner_check) {
  if (nblk < 1 || nkt < 1 || grid < 1 || !begin_out) return MK_E_INVALID;
  if ((unsigned long long)nblk * nkt * (grid + 1ull) >= (1ull << 32)) return MK_E_INVALID;
  const unsigned total = (unsigned)(nblk * nkt);
  for (int c = 0; c <= grid; ++c) begin_out[c] = mk::tile_begin(c, total, grid);
  int bad = 0;
  for (unsigned t = 0; t < total; ++t) {
    const int o = mk::tile_owner(t, total, grid);
    if (o < 0 || o >= grid || t < begin_out[o] || t >= begin_out[o + 1]) ++bad;
  }
  if (owner_check) *owner_check = bad;
  return 0;
}

int mk_debug_exchange_sequence(uint32_t total_before, uint32_t k, int world, int tokens, int cols, uint32_t* seq_out,
                               int64_t* first_word_out, int* stale_arrived_out) {
  if (k < 1 || world < 1 || tokens < 1 || cols < 1 || !seq_out) return MK_E_INVALID;
  const unsigned seq = mk::xchg_seq(total_before, k);
  *seq_out = seq;
  if (first_word_out) *first_word_out = (int64_t)mk::xchg_word(seq, world, tokens, cols, 0, 0, 0);
  if (stale_arrived_out) {
    // what the same half of the region held before: the exchanges two, four, ... steps back, or zeros
    int stale = 0;
    for (unsigned back = 2; back <= 64; back += 2) stale += mk::xchg_arrived(seq - back, seq) ? 1 : 0;
    *stale_arrived_out = stale;
  }
  return 0;
}

int mk_barrier_target_reached(uint32_t counter, uint32_t epoch, uint32_t arrivals_per_barrier) {
  // the comparison the device's grid barrier makes (modulo 2^32)
  return (int)(counter - epoch * arrivals_per_barrier) >= 0 ? 1 : 0;
}

// Everything of mk_compile that depends on the width a program is planned for (h->plan_tokens): the
// shared-memory carve-up, scratch, tensor maps, op descriptors and kernel parameters of the plan in
// h->plan.  `first`: also allocates the scheduler state the programs of a handle share.
static int compile_program(mk_handle* h, bool first) {
  const mk_config& cfg = h->cfg;
  cudaError_t ce;
  // 2. shared-memory carve-up: [weight ring: stages x (32 KB of weights + two activation
  // boxes of x_rows token rows)][x region: rows staged by the consumers for a fused input
  // norm, attention scratch][sums block of a tile: 128 x x_rows floats][small scratch]
  // [barriers, flags].  Above 8 tokens nothing is staged by the consumers and the sums
  // block shares the x region.
  const bool wide = h->plan_tokens > mk::kMaxTokGroup;
  const int nt = h->plan_tokens;
  const bool rows_mode = h->rows_mode;  // row-owner linears: resident token rows, no activation boxes
  const int x_rows = rows_mode ? 0 : (nt <= 8 ? 8 : (nt <= 16 ? 16 : (nt <= 32 ? 32 : 64)));
  const int stage_bytes = mk::kStageBytes + 2 * x_rows * 128;
  const int sums_bytes = rows_mode ? kRowsSumsBytes : mk::kTileRows * x_rows * 4;
  const int sums_sep = wide ? 0 : sums_bytes;
  const int tb_max = std::min(mk::kMaxTokGroup, nt);
  const int fixed0 = 1024 /*alignment slack*/ + sums_sep + kRedBytes + 1024 /*barriers, flags*/;
  // Measured on B200: a CTA whose shared memory (plus the 1 KB the system adds) stays within
  // the 164 KB carve-out leaves 92 KB of the SM's unified array to L1, and the whole kernel
  // runs about 8 % faster than with the next carve-out (196 KB, 60 KB of L1).
  const int want_stages = cfg.max_stages > 0 ? std::min(cfg.max_stages, 16) : 4;
  // (row-owner mode prefers two resident token rows and three stages to one row and four)
  int x_budget = rows_mode ? kRowsXBudget : kFastSmem - fixed0 - want_stages * stage_bytes;
  int x_bytes = std::max(cfg.max_num_pages * 4, wide ? sums_bytes : 0);
  int max_nblk = 1, n_linear = 0, min_tpp = rows_mode ? 2 : x_rows;
  bool has_moe = false;
  const int kpad_to = rows_mode ? mk::kRowsStageK : mk::kTileK;  // the staged rows are padded to whole stages
  for (int attempt = 0; attempt < 2; ++attempt) {
    bool fits = true;
    for (PlanOp& p : h->plan) {
      if (p.type != mk::OP_LINEAR || !(p.flags & (mk::F_NORM_IN | mk::F_ROWS))) continue;
      const int kp = (p.k + kpad_to - 1) / kpad_to * kpad_to;
      if ((x_budget - 16) / ((kp + 8) * 2) < 1) fits = false;
    }
    if (fits) break;
    x_budget = kMaxSmem - fixed0 - 3 * stage_bytes;  // a wide fused norm: give up the small carve-out
  }
  for (PlanOp& p : h->plan) {
    if (p.type == mk::OP_LINEAR) {
      max_nblk = std::max(max_nblk, (p.n + mk::kTileRows - 1) / mk::kTileRows);
      ++n_linear;
      if (wide && (p.flags & mk::F_NORM_IN)) return h->fail(MK_E_UNSUPPORTED, "rmsnorm_linear is only built for up to 8 batched tokens");
      if (!(p.flags & (mk::F_NORM_IN | mk::F_ROWS))) {
        // no fused norm: the input is read straight from the previous task's output, as
        // activation boxes that ride with the weight stages
        p.flags |= mk::F_XTILE;
        p.aux3 = x_rows;
        continue;
      }
      const int kp = (p.k + kpad_to - 1) / kpad_to * kpad_to;
      const int row_bytes = (kp + 8) * 2;
      int tpp = std::min(rows_mode ? std::min(2, nt) : tb_max, (x_budget - 16) / row_bytes);
      if (tpp < 1) return h->fail(MK_E_UNSUPPORTED, "K=%d is too wide for a fused input norm", p.k);
      p.aux3 = tpp;
      min_tpp = std::min(min_tpp, tpp);
      x_bytes = std::max(x_bytes, tpp * row_bytes + 16);
    } else if (p.type == mk::OP_MOE_LINEAR) {
      // a CTA stages the input rows of the pairs its share of the virtual row space (pairs x n rows) touches
      ++n_linear;
      has_moe = true;
      const int kp = (p.k + mk::kRowsStageK - 1) / mk::kRowsStageK * mk::kRowsStageK;
      const int64_t pairs = (int64_t)nt * p.aux0;
      const int64_t units = pairs * (p.n / mk::kUnitRows);
      const int g = (int)std::min<int64_t>(h->num_sms, units);
      const int64_t rows_per_cta = ((units + g - 1) / g) * mk::kUnitRows;
      int spans = (int)((rows_per_cta + p.n - 1) / p.n + 1);
      if (p.flags & mk::F_MOE_COMBINE) spans = std::max(spans, p.aux0);  // (the token's top-k input rows)
      if (spans > 8) return h->fail(MK_E_UNSUPPORTED, "moe linear: %d rows per expert are too few for the row-owner split", p.n);
      if (spans * (kp + 8) * 2 + 16 > x_budget) return h->fail(MK_E_UNSUPPORTED, "moe linear: K=%d is too wide", p.k);
      x_bytes = std::max(x_bytes, spans * (kp + 8) * 2 + 16);
    } else if (p.type == mk::OP_RMSNORM) {
      x_bytes = std::max(x_bytes, ((p.n + 63) / 64 * 64 + 8) * 2 + 16);
    } else if (p.type == mk::OP_ATTN) {
      // q heads and the new k (bf16), four combine slots of 4 heads x 128 floats, (max, sum) pairs, merge scratch
      x_bytes = std::max(x_bytes, 9 * 256 + 4 * 4 * (mk::kHeadDim + 2) * 4 + 2 * kAttnMaxChunks * 8 * 4 + 64 + 256);
      // above 16 tokens several (request, kv head) pairs run side by side in a CTA: q/k per group
      // (4 x 1280 B) and one combine slot per warp (8 x 4 heads x 128 floats + (max, sum) pairs)
      if (x_rows >= 32) x_bytes = std::max(x_bytes, 4 * 1280 + 8 * 4 * mk::kHeadDim * 4 + 8 * 4 * 2 * 4);
      // the tensor-core pass of the wider paths: q heads, new k and v, (warp x head) combine slots, page numbers
      if (!rows_mode) x_bytes = std::max(x_bytes, 10 * 256 + 8 * 4 * (mk::kHeadDim + 2) * 4 + 128 + 256);
    }
  }
  if (has_moe) x_bytes += 512;  // the expert ids of the pairs, for the producer (routing folded into the expert linear)
  x_bytes = (x_bytes + 1023) / 1024 * 1024;
  const int fixed = fixed0 + x_bytes;
  const int s_fast = (kFastSmem - fixed) / stage_bytes, s_max = (kMaxSmem - fixed) / stage_bytes;
  int stages;
  if (cfg.max_stages > 0) stages = std::min(s_max, want_stages);  // an explicit request wins
  else stages = std::min(s_fast, 4) >= 3 ? std::min(s_fast, 4) : std::min(s_max, 4);
  if (stages < 2) return h->fail(MK_E_UNSUPPORTED, "activations need %d bytes of shared memory: no room for the weight ring", x_bytes);
  mk::KParams& kp = h->kp;
  memset(&kp, 0, sizeof(kp));
  kp.num_stages = stages;
  kp.stage_bytes = stage_bytes;
  kp.x_rows = x_rows;
  kp.x_off = stages * stage_bytes;
  kp.x_bytes = x_bytes;
  kp.sums_off = wide ? kp.x_off : kp.x_off + x_bytes;
  kp.sums_stride = rows_mode ? 2 : x_rows;
  kp.red_off = kp.x_off + x_bytes + sums_sep;
  kp.bar_off = kp.red_off + kRedBytes;
  h->smem_bytes = kp.bar_off + 1024 + 1024;
  kp.path = rows_mode ? mk::PATH_ROWS : (x_rows >= 32 ? mk::PATH_UMMA : mk::PATH_TILES);
  kp.rank = cfg.rank;
  kp.world = cfg.world_size;
  kp.cluster = 1;
  const int per_sm = mk_kernel_max_ctas_per_sm(&kp, h->smem_bytes);
  if (per_sm < 1) return h->fail(MK_E_CUDA, "the megakernel does not fit on an SM with %d bytes of shared memory", h->smem_bytes);
  h->grid = h->num_sms;
  if (cfg.num_workers > 0) h->grid = std::min(h->grid, cfg.num_workers);
  // Grid barrier shape: hierarchical (cluster-first) when asked for and every cluster of the grid
  // can be resident at once; otherwise flat.
  if (cfg.cluster_size == 2 || cfg.cluster_size == 4) {
    if (cfg.world_size > 1) return h->fail(MK_E_UNSUPPORTED, "the cluster-first grid barrier is only built for single-GPU launches");
    const int cs = cfg.cluster_size;
    const int fit = mk_kernel_max_clusters(kp.path, h->smem_bytes, cs, h->grid / cs * cs);
    if (fit >= 1) {
      kp.cluster = cs;
      h->grid = std::min(h->grid / cs, fit) * cs;
    }
  } else if (cfg.cluster_size > 1) {
    return h->fail(MK_E_INVALID, "cluster_size must be 0, 1, 2 or 4");
  }
  kp.bar_epoch0 = cfg.test_barrier_epoch;
  h->max_nblk = max_nblk;
  // row-owner LM head: one (max, index) partial per CTA that owns rows
  for (size_t i = 0; i < h->plan.size(); ++i) {
    PlanOp& po = h->plan[i];
    if (po.type == mk::OP_LINEAR && (po.flags & mk::F_ROWS) && (po.flags & mk::F_ARGMAX)) {
      po.amax_n = std::min(h->grid, (po.n + mk::kUnitRows - 1) / mk::kUnitRows);
      if (i + 1 < h->plan.size() && h->plan[i + 1].type == mk::OP_ARGMAX_REDUCE) h->plan[i + 1].amax_n = po.amax_n;
    }
  }

  // Tagged activations (row-owner programs).  Where an op's input is the output of the op right before it,
  // and both are row-owner linears or attention, the producer also stores its outputs as 8-byte words
  // {two bf16 columns, tag} and the consumer polls the words it reads instead of waiting at a grid barrier.
  // Why dropping the barrier is safe: a CTA reads a buffer in an op only to produce outputs of that op, and
  // every consumer waits for all the outputs it reads (a linear for the whole row, the attention tasks between
  // them for every column of the QKV row), so whoever overwrites a buffer later has, through the chain of
  // consumers, waited for everything its earlier readers produced.  A residual is read from the words of its
  // own producer, or must be older than a barrier that is kept.
  std::map<int, size_t> ll_off;  // tensor -> byte offset of its words in the program's arena
  size_t ll_bytes = 0;
  if (rows_mode && !has_moe && kp.cluster == 1 && !(cfg.debug_flags & 16)) {
    auto ll_tensor = [&](int id) {
      if (!ll_off.count(id)) {
        const Tensor& t = h->tensors[id];
        ll_off[id] = ll_bytes;
        ll_bytes += ((size_t)t.dims[0] * (size_t)t.strides[0] * 4 + 255) / 256 * 256;
      }
    };
    auto row_linear = [&](const PlanOp& q) { return q.type == mk::OP_LINEAR && (q.flags & mk::F_ROWS) && q.n % 8 == 0; };
    auto plain_2d = [&](int id) {
      if (id < 0) return false;
      const Tensor& t = h->tensors[id];
      return t.ndim == 2 && t.dtype == MK_BF16 && t.strides[1] == 1 && t.strides[0] % 8 == 0;
    };
    // what the two tagged-input stagings of the kernel cover: a fused norm with at most four 16-byte
    // vectors per lane, or no norm and at most 24 stages of k
    auto stage_ok = [&](const PlanOp& q) {
      const int nkt = (q.k + mk::kRowsStageK - 1) / mk::kRowsStageK;
      const int wpr = q.aux3 <= 1 ? 8 : 4;
      if (q.flags & mk::F_NORM_IN) return nkt * (mk::kRowsStageK / 8) <= 128 * wpr;
      return nkt <= 24 && q.aux3 <= 2;
    };
    std::map<int, int> reduced_by;  // tensor parallelism: virtual tensor -> the op that adds its exchange up into tagged words
    for (size_t i = 1; i < h->plan.size(); ++i) {
      PlanOp& cur = h->plan[i];
      PlanOp& prev = h->plan[i - 1];
      if (cfg.world_size > 1 && row_linear(cur) && plain_2d(cur.in) && stage_ok(cur) && !(cur.flags & mk::F_SYNC_BEFORE) &&
          (cur.flags & mk::F_GATHER_IN)) {
        // every CTA adds up a slice of the exchange, all of them read the sums as tagged words
        cur.flags = (cur.flags & ~mk::F_GATHER_IN) | mk::F_XRED | mk::F_LL_IN;
        cur.ll_in_op = (int)i;
        ll_tensor(cur.in);
        reduced_by[cur.in] = (int)i;
        continue;
      }
      if (cfg.world_size > 1 && row_linear(cur) && (cur.flags & mk::F_GATHER_RES) && cur.res >= 0 && reduced_by.count(cur.res) &&
          plain_2d(cur.res)) {
        // the residual of a pushing linear: the sums an earlier op of this iteration left as tagged words
        cur.flags = (cur.flags & ~mk::F_GATHER_RES) | mk::F_LL_RES;
        cur.ll_res_op = reduced_by[cur.res];
      }
      if (!(cur.flags & mk::F_SYNC_BEFORE) || cur.in < 0 || cur.in != prev.out || !plain_2d(cur.in)) continue;
      bool ok = false;
      if (row_linear(cur) && !(cur.flags & mk::F_GATHER_IN)) {
        ok = ((row_linear(prev) && !(prev.flags & (mk::F_PUSH | mk::F_ARGMAX))) || prev.type == mk::OP_ATTN) && stage_ok(cur);
      } else if (cur.type == mk::OP_ATTN) {
        ok = row_linear(prev) && !(prev.flags & (mk::F_PUSH | mk::F_ARGMAX | mk::F_SILU_MUL));
      }
      if (!ok) continue;
      int res_op = -1;
      if (cur.res >= 0 && !(cur.flags & mk::F_GATHER_RES)) {
        int wq = -1;
        for (int q = (int)i - 1; q >= 0; --q)
          if (h->plan[q].out == cur.res) {
            wq = q;
            break;
          }
        if (wq >= 0) {
          if ((h->plan[wq].flags & mk::F_LL_OUT) && plain_2d(cur.res)) {
            res_op = wq;
          } else {
            bool fenced = false;  // a kept barrier between the residual's writer and this op
            for (int b = wq + 1; b < (int)i; ++b) fenced = fenced || (h->plan[b].flags & mk::F_SYNC_BEFORE);
            if (!fenced) continue;
          }
        }
      }
      cur.flags = (cur.flags & ~mk::F_SYNC_BEFORE) | mk::F_LL_IN;
      cur.ll_in_op = (int)i - 1;
      prev.flags |= mk::F_LL_OUT;
      ll_tensor(cur.in);
      if (res_op >= 0) {
        cur.flags |= mk::F_LL_RES;
        cur.ll_res_op = res_op;
      }
    }
  }
  // the attention chunks' partials as tagged words too (merged without a counter), in the same arena.  (The
  // chunks of a pair must be tasks of one round, or of consecutive CTAs across two: at least 64 CTAs.)
  size_t ll_part_off = 0;
  bool ll_part = false;
  for (const PlanOp& po : h->plan) ll_part = ll_part || (po.type == mk::OP_ATTN && (po.flags & mk::F_LL_OUT));
  ll_part = ll_part && h->grid >= 64;
  if (ll_part) {
    int hkv = 1, qpk = 2;
    for (const PlanOp& po : h->plan)
      if (po.type == mk::OP_ATTN) {
        hkv = std::max(hkv, po.aux0);
        qpk = std::max(qpk, po.aux1 / po.aux0);
      }
    ll_part_off = ll_bytes;
    ll_bytes += ((size_t)h->plan_tokens * hkv * kAttnMaxChunks * qpk * (mk::kHeadDim + 2) * 8 + 255) / 256 * 256;
  }
  h->ll_buf = nullptr;
  h->ll_bytes = ll_bytes;
  if (ll_bytes > 0) {
    if (int e = h->dmalloc(&h->ll_buf, ll_bytes)) return e;
  }
  kp.attn_part_ll = ll_part ? (uint2*)((char*)h->ll_buf + ll_part_off) : nullptr;

  // 3. scratch and state
  const int G = h->grid;
  const int groups = (h->plan_tokens + min_tpp - 1) / min_tpp;
  void* p = nullptr;
  if (int e = h->dmalloc(&p, (size_t)groups * G * 2 * mk::kTileRows * kp.sums_stride * 4)) return e;
  kp.partial = (float*)p;
  const size_t piece_count_bytes = (size_t)groups * max_nblk * 4;
  h->piece_count_bytes = piece_count_bytes;
  if (int e = h->dmalloc(&p, h->piece_count_bytes)) return e;
  kp.piece_count = (unsigned*)p;
  kp.piece_stride = max_nblk;
  int max_hkv = 1, max_qpk = 2;
  for (const PlanOp& po : h->plan)
    if (po.type == mk::OP_ATTN) {
      max_hkv = std::max(max_hkv, po.aux0);
      max_qpk = std::max(max_qpk, po.aux1 / po.aux0);
    }
  kp.attn_max_chunks = kAttnMaxChunks;
  if (int e = h->dmalloc(&p, (size_t)h->plan_tokens * max_hkv * kAttnMaxChunks * max_qpk * (mk::kHeadDim + 2) * 4)) return e;
  kp.attn_part = (float*)p;
  h->attn_count_bytes = (size_t)h->plan_tokens * max_hkv * 4;
  if (int e = h->dmalloc(&p, h->attn_count_bytes)) return e;
  kp.attn_count = (unsigned*)p;
  if (first) {
    if (int e = h->dmalloc(&p, (size_t)cfg.max_num_batched_requests * 4)) return e;
    kp.request_ids = (int*)p;
    if (int e = h->dmalloc(&p, (size_t)cfg.max_num_pages * 4)) return e;
    kp.page_queue = (int*)p;
    if (int e = h->dmalloc(&p, 256)) return e;
    kp.sched = (int*)p;
    kp.grid_bar = (unsigned*)p + 16;
    kp.ctrl = (int*)p + 20;
    kp.abort_flag = (int*)p + 17;  // beside the barrier counter: one 8-byte load polls both
    kp.status = (int*)p + 32;
    if (int e = h->dmalloc(&p, (size_t)kMaxStepTimes * 16)) return e;
    kp.step_times = (unsigned long long*)p;
  } else {
    // the scheduler's state is shared by the programs of a handle
    const mk::KParams& k0 = h->prog[0].kp;
    kp.request_ids = k0.request_ids;
    kp.page_queue = k0.page_queue;
    kp.sched = k0.sched;
    kp.grid_bar = k0.grid_bar;
    kp.ctrl = k0.ctrl;
    kp.abort_flag = k0.abort_flag;
    kp.status = k0.status;
    kp.step_times = k0.step_times;
  }
  kp.max_step_times = kMaxStepTimes;

  // 4. the program
  std::vector<mk::OpDesc> descs(h->plan.size());
  std::vector<CUtensorMap> maps;
  std::vector<int> map_of(h->plan.size(), -1), xmap_of(h->plan.size(), -1);
  EncodeTiledFn encode = get_encode_fn();
  if (n_linear && !encode) return h->fail(MK_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  auto tp = [&](int id) -> void* { return id >= 0 ? h->tensors[id].ptr : nullptr; };
  auto ld = [&](int id) -> int { return id >= 0 ? (int)h->tensors[id].strides[0] : 0; };
  h->weight_bytes = 0;
  float* last_amax_val = nullptr;
  int* last_amax_idx = nullptr;
  // mixture of experts: the routing tables [tokens, top-k] (renormalised softmax weight, expert id)
  float* route_w = nullptr;
  int* route_idx = nullptr;
  if (has_moe) {
    void* q = nullptr;
    if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * 32 * 4)) return e;
    route_w = (float*)q;
    if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * 32 * 4)) return e;
    route_idx = (int*)q;
  }
  for (size_t i = 0; i < h->plan.size(); ++i) {
    const PlanOp& po = h->plan[i];
    mk::OpDesc& d = descs[i];
    memset(&d, 0, sizeof(d));
    d.type = po.type;
    d.flags = po.flags;
    d.n = po.n;
    d.k = po.k;
    d.aux0 = po.aux0; d.aux1 = po.aux1; d.aux2 = po.aux2; d.aux3 = po.aux3;
    d.in = tp(po.in);
    d.w = tp(po.w);
    d.norm_w = tp(po.norm_w);
    d.res = tp(po.res);
    d.out = tp(po.out);
    d.ld_in = ld(po.in);
    d.ld_out = ld(po.out);
    d.ld_res = ld(po.res);
    d.amax_n = po.amax_n;
    d.ll_in_op = po.ll_in_op;
    d.ll_res_op = po.ll_res_op;
    if (po.flags & mk::F_LL_IN) d.ll_in = (char*)h->ll_buf + ll_off.at(po.in);
    if (po.flags & mk::F_LL_OUT) d.ll_out = (char*)h->ll_buf + ll_off.at(po.out);
    if (po.flags & mk::F_LL_RES) d.ll_res = (char*)h->ll_buf + ll_off.at(po.res);
    if (po.type == mk::OP_EMBED) {
      d.ld_res = ld(po.w);
      d.ld_in = (int)h->tensors[po.in].strides[0];
    } else if (po.type == mk::OP_LINEAR) {
      const Tensor& w = h->tensors[po.w];
      if (po.flags & mk::F_ROWS) {
        // four maps, for chunks of 8, 16, 24 and 32 rows: box = 64 k-elements x that many rows
        const int units = (po.n + mk::kUnitRows - 1) / mk::kUnitRows;
        d.nblk = units;
        d.ld_out2 = (int)w.strides[0];  // the weight pitch, for the L2 look-ahead
        d.nkt = (po.k + mk::kRowsStageK - 1) / mk::kRowsStageK;
        if (((uintptr_t)w.ptr) & 15) return h->fail(MK_E_INVALID, "weight %s is not 16-byte aligned", w.name.c_str());
        map_of[i] = (int)maps.size();
        for (int rows = mk::kUnitRows; rows <= mk::kChunkRows; rows += mk::kUnitRows) {
          CUtensorMap m;
          cuuint64_t gdim[2] = {(cuuint64_t)po.k, (cuuint64_t)po.n};
          cuuint64_t gstr[1] = {(cuuint64_t)w.strides[0] * 2};
          cuuint32_t box[2] = {(cuuint32_t)mk::kBoxK, (cuuint32_t)rows};
          cuuint32_t estr[2] = {1, 1};
          CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w.ptr, gdim, gstr, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
          if (r != CUDA_SUCCESS) return h->fail(MK_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %s [%d x %d]", (int)r, w.name.c_str(), po.n, po.k);
          maps.push_back(m);
        }
        h->weight_bytes += (int64_t)units * mk::kUnitRows * d.nkt * mk::kRowsStageK * 2;
        if (po.flags & mk::F_ARGMAX) {
          void* q = nullptr;
          if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
          d.amax_val = last_amax_val = (float*)q;
          if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
          d.amax_idx = last_amax_idx = (int*)q;
        }
        continue;
      }
      d.nblk = (po.n + mk::kTileRows - 1) / mk::kTileRows;
      d.nkt = (po.k + mk::kTileK - 1) / mk::kTileK;
      CUtensorMap m;
      cuuint64_t gdim[2] = {(cuuint64_t)po.k, (cuuint64_t)po.n};
      cuuint64_t gstr[1] = {(cuuint64_t)w.strides[0] * 2};
      cuuint32_t box[2] = {(cuuint32_t)mk::kBoxK, (cuuint32_t)mk::kTileRows};
      cuuint32_t estr[2] = {1, 1};
      if (((uintptr_t)w.ptr) & 15) return h->fail(MK_E_INVALID, "weight %s is not 16-byte aligned", w.name.c_str());
      CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w.ptr, gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return h->fail(MK_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %s [%d x %d]", (int)r, w.name.c_str(), po.n, po.k);
      map_of[i] = (int)maps.size();
      maps.push_back(m);
      if (po.flags & mk::F_XTILE) {
        const Tensor& x = h->tensors[po.in];
        CUtensorMap mx;
        cuuint64_t xdim[2] = {(cuuint64_t)po.k, (cuuint64_t)x.dims[0]};
        cuuint64_t xstr[1] = {(cuuint64_t)x.strides[0] * 2};
        cuuint32_t xbox[2] = {(cuuint32_t)mk::kBoxK, (cuuint32_t)kp.x_rows};
        if ((((uintptr_t)x.ptr) & 15) || (x.strides[0] % 8)) return h->fail(MK_E_INVALID, "input %s of a linear must be 16-byte aligned with a pitch multiple of 8", x.name.c_str());
        r = encode(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x.ptr, xdim, xstr, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return h->fail(MK_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for the input %s", (int)r, x.name.c_str());
        xmap_of[i] = (int)maps.size();
        maps.push_back(mx);
      }
      if ((unsigned long long)d.nblk * d.nkt * (G + 1ull) >= (1ull << 32))
        return h->fail(MK_E_UNSUPPORTED, "%s has too many weight tiles for 32-bit tile arithmetic", w.name.c_str());
      h->weight_bytes += (int64_t)d.nblk * d.nkt * mk::kStageBytes;
      if (po.flags & mk::F_ARGMAX) {
        void* q = nullptr;
        if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
        d.amax_val = last_amax_val = (float*)q;
        if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
        d.amax_idx = last_amax_idx = (int*)q;
      }
    } else if (po.type == mk::OP_MOE_LINEAR) {
      // the [experts, n, K] weight as one 2-D [experts * n, K] tensor: four maps, for chunks of 8, 16, 24 and 32 rows
      const Tensor& w = h->tensors[po.w];
      const Tensor &ti = h->tensors[po.in], &to = h->tensors[po.out];
      d.ld_in = (int)ti.strides[ti.ndim - 2];
      d.ld_out = (int)to.strides[to.ndim - 2];
      d.nkt = (po.k + mk::kRowsStageK - 1) / mk::kRowsStageK;
      d.amax_idx = route_idx;
      d.amax_val = route_w;
      if (((uintptr_t)w.ptr) & 15) return h->fail(MK_E_INVALID, "weight %s is not 16-byte aligned", w.name.c_str());
      map_of[i] = (int)maps.size();
      for (int rows = mk::kUnitRows; rows <= mk::kChunkRows; rows += mk::kUnitRows) {
        CUtensorMap m;
        cuuint64_t gdim[2] = {(cuuint64_t)po.k, (cuuint64_t)((int64_t)po.aux1 * po.n)};
        cuuint64_t gstr[1] = {(cuuint64_t)po.k * 2};
        cuuint32_t box[2] = {(cuuint32_t)mk::kBoxK, (cuuint32_t)rows};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w.ptr, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return h->fail(MK_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %s", (int)r, w.name.c_str());
        maps.push_back(m);
      }
      h->weight_bytes += (int64_t)po.aux0 * po.n * d.nkt * mk::kRowsStageK * 2;  // per token
    } else if (po.type == mk::OP_MOE_ROUTE) {
      d.amax_val = route_w;
      d.amax_idx = route_idx;
    } else if (po.type == mk::OP_MOE_COMBINE) {
      const Tensor& ti = h->tensors[po.in];
      d.ld_in = (int)ti.strides[ti.ndim - 2];
      d.amax_val = route_w;
    } else if (po.type == mk::OP_SILU_MUL && po.aux1 > 0) {
      const Tensor &ti = h->tensors[po.in], &to = h->tensors[po.out];
      d.ld_in = (int)ti.strides[ti.ndim - 2];
      d.ld_out = (int)to.strides[to.ndim - 2];
    } else if (po.type == mk::OP_ATTN) {
      d.k_cache = tp(po.kc);
      d.v_cache = tp(po.vc);
      d.q_norm_w = tp(po.qn);
      d.k_norm_w = tp(po.kn);
      d.cos = tp(po.cos);
      d.sin = tp(po.sin);
    } else if (po.type == mk::OP_ARGMAX_PARTIAL) {
      void* q = nullptr;
      if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
      d.amax_val = last_amax_val = (float*)q;
      if (int e = h->dmalloc(&q, (size_t)h->plan_tokens * po.amax_n * 4)) return e;
      d.amax_idx = last_amax_idx = (int*)q;
    } else if (po.type == mk::OP_ARGMAX_REDUCE) {
      d.amax_val = last_amax_val;
      d.amax_idx = last_amax_idx;
      d.ld_out = (int)h->tensors[po.out].strides[0];
    }
  }
  if (!maps.empty()) {
    if (int e = h->dmalloc(&p, maps.size() * sizeof(CUtensorMap), false)) return e;
    if ((ce = cudaMemcpy(p, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice)) != cudaSuccess)
      return h->cuda_fail(ce, "tensor map upload");
    for (size_t i = 0; i < descs.size(); ++i)
      if (map_of[i] >= 0) descs[i].tmap_w = (const char*)p + (size_t)map_of[i] * sizeof(CUtensorMap);
    for (size_t i = 0; i < descs.size(); ++i)
      if (xmap_of[i] >= 0) descs[i].tmap_x = (const char*)p + (size_t)xmap_of[i] * sizeof(CUtensorMap);
  }
  if (int e = h->dmalloc(&p, descs.size() * sizeof(mk::OpDesc), false)) return e;
  if ((ce = cudaMemcpy(p, descs.data(), descs.size() * sizeof(mk::OpDesc), cudaMemcpyHostToDevice)) != cudaSuccess)
    return h->cuda_fail(ce, "program upload");
  kp.ops = (const mk::OpDesc*)p;
  kp.num_ops = (int)descs.size();

  kp.mode = cfg.mode;
  kp.numerics = cfg.numerics;
  kp.rank = cfg.rank;
  kp.world = cfg.world_size;
  kp.step = (int*)h->meta[0];
  kp.tokens = (long long*)h->meta[1];
  kp.input_tokens = (long long*)h->meta[2];
  kp.output_tokens = (long long*)h->meta[3];
  kp.num_new_tokens = (int*)h->meta[4];
  kp.prompt_lengths = (int*)h->meta[5];
  kp.qo_indptr = (int*)h->meta[6];
  kp.kv_indptr = (int*)h->meta[7];
  kp.kv_indices = (int*)h->meta[8];
  kp.kv_last_page_len = (int*)h->meta[9];
  kp.max_seq_len = cfg.max_seq_length;
  kp.max_reqs = cfg.max_num_batched_requests;
  kp.max_tokens = cfg.max_num_batched_tokens;  // the scheduler's budget per iteration (tok_lo/tok_hi say what this program serves)
  kp.max_tokens_per_req = cfg.max_tokens_per_request > 0 ? cfg.max_tokens_per_request : cfg.max_num_batched_tokens;
  kp.max_pages = cfg.max_num_pages;
  kp.page_size = cfg.page_size;
  kp.page_shift = 0;
  while ((1 << kp.page_shift) < cfg.page_size) ++kp.page_shift;
  kp.total_requests = (int)h->total_requests;
  kp.eos = cfg.eos_token_id;
  kp.max_iters = cfg.max_iterations;
  kp.timeout_ns = (unsigned long long)cfg.timeout_ms * 1000000ull;
  if (xchg_bytes(h) > 0) {
    if (!h->xchg_ready) return h->fail(MK_E_STATE, "the graph has allreduce layers: exchange handles with mk_comm_prepare / mk_comm_connect before mk_compile");
    for (int r = 0; r < cfg.world_size; ++r) kp.xchg[r] = (unsigned char*)h->xchg_peer[r];
    kp.xchg_tokens = h->xchg_tokens;
    kp.xchg_cols = h->xchg_cols;
    kp.xchg_amax_word = h->xchg_amax_word;
  }
  kp.trace_op = -1;
  kp.debug_flags = cfg.debug_flags;
  // L2 look-ahead of the weight stream, in 32 KB stages: on by default (512 KB per CTA, the
  // measured optimum with evict-first weight loads) for a row-owner program whose ops all keep their grid
  // barriers, off elsewhere (it measured slower there); prefetch_kb > 0 sets it, < 0 turns it off
  kp.has_moe = has_moe ? 1 : 0;
  // (no look-ahead with expert layers: which weights come next is only known after routing)
  // (with tagged activations the gaps between the ops are short and the look-ahead only competes with the ring:
  // measured 3.51 against 3.56 ms per step at context 100 and 3.84 against 3.97 at context 600 with it off)
  const int pf_kb = has_moe ? 0 : (cfg.prefetch_kb != 0 ? cfg.prefetch_kb : ((h->rows_mode && h->ll_bytes == 0) ? 512 : 0));
  kp.prefetch_tiles = pf_kb > 0 ? std::max(1, pf_kb * 1024 / mk::kStageBytes) : 0;
  if (h->prof_ptr && first) {  // (the trace describes the primary program's ops)
    const int64_t need = ((int64_t)descs.size() + 1) * G * 4 + (int64_t)G * 16;
    if (h->prof_entries < need) return h->fail(MK_E_INVALID, "profiler buffer has %lld words, the trace needs %lld", (long long)h->prof_entries, (long long)need);
    kp.prof = (unsigned long long*)h->prof_ptr;
    kp.trace_op = cfg.trace_op - 1;
  }
  return 0;
}

int mk_compile(mk_handle* h) {
  if (!h) return MK_E_INVALID;
  if (h->compiled) return h->fail(MK_E_STATE, "already compiled");
  if (!h->meta_set) return h->fail(MK_E_STATE, "mk_set_meta must be called before mk_compile");
  if (int e = mk_plan(h)) return e;
  const mk_config& cfg = h->cfg;
  cudaError_t ce;
  int dev = cfg.device;
  if (dev < 0) {
    if ((ce = cudaGetDevice(&dev)) != cudaSuccess) return h->cuda_fail(ce, "cudaGetDevice (is a CUDA device present?)");
  } else if ((ce = cudaSetDevice(dev)) != cudaSuccess) {
    return h->cuda_fail(ce, "cudaSetDevice");
  }
  cudaDeviceProp prop;
  if ((ce = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return h->cuda_fail(ce, "cudaGetDeviceProperties");
  if (prop.major != 10) return h->fail(MK_E_UNSUPPORTED, "this library only runs on sm_100 (found sm_%d%d)", prop.major, prop.minor);
  if (!prop.cooperativeLaunch) return h->fail(MK_E_UNSUPPORTED, "device lacks cooperative launch");
  h->num_sms = prop.multiProcessorCount;

  // 1. runtime-owned tensors (shuffles are filled below)
  for (auto& t : h->tensors)
    if (t.owned && !t.ptr)
      if (int e = h->dmalloc(&t.ptr, t.alloc_bytes())) return e;
  for (auto& t : h->tensors)
    if (!t.src.empty())
      if (int e = materialise_shuffle(h, t)) return e;
  if ((ce = cudaDeviceSynchronize()) != cudaSuccess) return h->cuda_fail(ce, "shuffle copies");

  // 2. the programs
  const bool two = two_programs(cfg);
  if (two && cfg.cluster_size > 1)
    return h->fail(MK_E_UNSUPPORTED, "cluster_size needs max_num_batched_tokens == max_num_batched_requests (one program)");
  h->nprog = 0;
  if (int e = compile_program(h, true)) return e;
  h->prog[0].plan = h->plan; h->prog[0].rows_mode = h->rows_mode; h->prog[0].max_tokens = h->plan_tokens;
  h->prog[0].kp = h->kp; h->prog[0].smem_bytes = h->smem_bytes; h->prog[0].weight_bytes = h->weight_bytes;
  h->prog[0].max_nblk = h->max_nblk;
  h->prog[0].attn_count_bytes = h->attn_count_bytes; h->prog[0].piece_count_bytes = h->piece_count_bytes;
  h->prog[0].ll_buf = h->ll_buf; h->prog[0].ll_bytes = h->ll_bytes;
  h->nprog = 1;
  if (two) {
    h->plan_tokens = cfg.max_num_batched_tokens;
    h->force_interleave = h->prog[0].rows_mode ? 4 : 64;
    if (int e = plan_graph(h)) return e;   // (same fusion decisions where they do not depend on the width)
    if (int e = compile_program(h, false)) return e;
    h->prog[1].plan = h->plan; h->prog[1].rows_mode = h->rows_mode; h->prog[1].max_tokens = h->plan_tokens;
    h->prog[1].kp = h->kp; h->prog[1].smem_bytes = h->smem_bytes; h->prog[1].weight_bytes = h->weight_bytes;
    h->prog[1].max_nblk = h->max_nblk;
    h->prog[1].attn_count_bytes = h->attn_count_bytes; h->prog[1].piece_count_bytes = h->piece_count_bytes;
    h->prog[1].ll_buf = h->ll_buf; h->prog[1].ll_bytes = h->ll_bytes;
    h->force_interleave = 0;
    h->nprog = 2;
    h->prog[0].kp.tok_lo = 1;
    h->prog[0].kp.tok_hi = h->prog[0].max_tokens;
    h->prog[1].kp.tok_lo = h->prog[0].max_tokens + 1;
    h->prog[1].kp.tok_hi = h->prog[1].max_tokens;
    // the handle's own copies describe the primary program again
    h->plan = h->prog[0].plan; h->rows_mode = h->prog[0].rows_mode; h->kp = h->prog[0].kp;
    h->smem_bytes = h->prog[0].smem_bytes; h->weight_bytes = h->prog[0].weight_bytes; h->max_nblk = h->prog[0].max_nblk;
    h->plan_tokens = h->prog[0].max_tokens;
  } else {
    h->prog[0].kp.tok_lo = 1;
    h->prog[0].kp.tok_hi = 1 << 30;
    h->kp = h->prog[0].kp;
  }
  h->cur_prog = 0;
  h->compiled = true;
  if (cfg.mode == MK_MODE_OFFLINE) return mk_init_requests(h, nullptr);
  return 0;
}

int mk_init_requests(mk_handle* h, void* stream) {
  if (!h) return MK_E_INVALID;
  if (!h->compiled) return h->fail(MK_E_STATE, "not compiled");
  if (h->cfg.mode != MK_MODE_OFFLINE) return 0;
  int e = mk_kernel_init_state(&h->kp, stream);
  if (e) return h->cuda_fail((cudaError_t)e, "init_state");
  cudaError_t ce = cudaStreamSynchronize((cudaStream_t)stream);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "init_state sync");
  return 0;
}

// One kernel of a generation call: the program's counters and the launch state are reset, then the
// persistent kernel of that program is launched.
static int launch_program(mk_handle* h, int idx, void* stream) {
  Program& P = h->prog[idx];
  cudaStream_t s = (cudaStream_t)stream;
  // grid barrier, control word, abort flag and status live in one 256-byte block behind sched[0..15]
  cudaError_t ce = cudaMemsetAsync((char*)P.kp.sched + 64, 0, 192, s);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  if (P.kp.bar_epoch0 != 0) {
    // (tests) the counter starts where barrier number bar_epoch0 has just been passed
    const unsigned start = P.kp.bar_epoch0 * (unsigned)(h->grid / std::max(1, P.kp.cluster));
    ce = cudaMemcpyAsync(P.kp.grid_bar, &start, 4, cudaMemcpyHostToDevice, s);
    if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  }
  // a launch that aborted may have left the arrival counters of its attention chunks and of its
  // split-k pieces half-way: a finisher that gave up clears its counter while late pieces still add to it
  ce = cudaMemsetAsync(P.kp.attn_count, 0, P.attn_count_bytes, s);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  ce = cudaMemsetAsync(P.kp.piece_count, 0, P.piece_count_bytes, s);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  if (P.ll_bytes > 0) {  // tags restart with every kernel: no word of an earlier one may look valid
    ce = cudaMemsetAsync(P.ll_buf, 0, P.ll_bytes, s);
    if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  }
  // exchange sequence numbers continue where the last kernel stopped (mk_wait adds what it executed)
  P.kp.xchg_seq_base = h->xchg_total;
  int e = mk_kernel_launch(&P.kp, h->grid, P.smem_bytes, stream);
  if (e) return h->cuda_fail((cudaError_t)e, "cooperative launch");
  return 0;
}

int mk_launch_async(mk_handle* h, void* stream) {
  if (!h) return MK_E_INVALID;
  if (!h->compiled) return h->fail(MK_E_STATE, "not compiled");
  if (h->in_flight) return h->fail(MK_E_STATE, "the previous launch has not been waited for (mk_wait)");
  if (h->poisoned)
    return h->fail(MK_E_STATE, "an earlier tensor-parallel launch aborted: the ranks' exchange sequence numbers may "
                               "differ; finalize this handle on every rank and build a new one");
  // a generation call starts with no iteration handed over and none completed (sched[5..7])
  cudaError_t ce = cudaMemsetAsync(h->prog[0].kp.sched + 5, 0, 12, (cudaStream_t)stream);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "state reset");
  if (int e = launch_program(h, h->cur_prog, stream)) return e;
  h->launched = true;
  h->in_flight = true;
  return 0;
}

int mk_wait(mk_handle* h, void* stream) {
  if (!h) return MK_E_INVALID;
  if (!h->launched) return h->fail(MK_E_STATE, "nothing launched");
  while (true) {
    cudaError_t ce = cudaStreamSynchronize((cudaStream_t)stream);
    h->in_flight = false;
    if (ce != cudaSuccess) return h->cuda_fail(ce, "megakernel");
    int st[24];
    ce = cudaMemcpy(st, h->prog[0].kp.abort_flag, sizeof(int) * 24, cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return h->cuda_fail(ce, "status readback");
    if (h->cfg.world_size > 1) {
      int done = 0;
      ce = cudaMemcpy(&done, h->prog[0].kp.sched + 6, 4, cudaMemcpyDeviceToHost);
      if (ce != cudaSuccess) return h->cuda_fail(ce, "status readback");
      h->xchg_total += (unsigned)done;
    }
    if (st[0] != 0) {
      static const char* names[] = {"ok", "grid barrier timed out", "weight stage never arrived", "weight ring never drained",
                                    "producer never got the next iteration", "peer never arrived", "token id out of range",
                                    "out of KV pages", "a peer rank never delivered its allreduce share",
                                    "an op's tagged input never arrived"};
      const int* s = st + 15;  // status sits 15 words behind the abort flag
      const int code = s[0];
      if (h->cfg.world_size > 1) h->poisoned = true;
      return h->fail(MK_E_DEVICE, "megakernel aborted: %s (code %d) at cta %d op %d iteration %d detail %d/%d thread %d",
                     (code >= 0 && code < 10) ? names[code] : "?", code, s[1], s[2], s[3], s[4], s[5], s[6]);
    }
    // ctrl[0] (3 words behind the abort flag) == -2: the kernel prepared an iteration that belongs to the
    // handle's other program and ended; that program takes over on the same stream
    if (st[3] != -2 || h->nprog < 2) return 0;
    h->cur_prog ^= 1;
    if (int e = launch_program(h, h->cur_prog, stream)) return e;
    h->in_flight = true;
  }
}

int mk_launch(mk_handle* h, void* stream) {
  if (int e = mk_launch_async(h, stream)) return e;
  return mk_wait(h, stream);
}

int mk_get_event_timing(mk_handle* h, uint64_t* buf, int max_entries) {
  if (!h || !buf || max_entries < 0) return MK_E_INVALID;
  if (!h->compiled) return h->fail(MK_E_STATE, "not compiled");
  int iters = 0;
  cudaError_t ce = cudaMemcpy(&iters, h->kp.sched + 3, 4, cudaMemcpyDeviceToHost);
  if (ce != cudaSuccess) return h->cuda_fail(ce, "timing readback");
  int n = std::min(std::min(iters + 1, max_entries), h->kp.max_step_times);
  if (n > 0) {
    ce = cudaMemcpy(buf, h->kp.step_times, (size_t)n * 16, cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return h->cuda_fail(ce, "timing readback");
  }
  return n;
}

int mk_finalize(mk_handle* h) {
  if (!h) return MK_E_INVALID;
  for (int r = 0; r < 8; ++r)
    if (h->xchg_peer[r] && h->xchg_peer[r] != h->xchg_local) cudaIpcCloseMemHandle(h->xchg_peer[r]);
  for (void* p : h->allocs) cudaFree(p);
  delete h;
  return 0;
}

}  // extern "C"
