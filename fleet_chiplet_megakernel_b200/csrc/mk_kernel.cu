// The persistent decode megakernel for sm_100a.
//
// One cooperative launch runs a whole generation.  Every SM hosts one CTA of
// nine warps: warp 8 is a TMA producer that streams this CTA's share of every
// linear layer's weights (128x64 bf16 tiles, 128-byte swizzle) into a ring of
// shared-memory stages, running ahead of the eight consumer warps across op
// boundaries (weights have no dependencies).  The consumer warps walk the
// program: wait at a grid barrier where an op reads what other CTAs wrote, do
// the op's share of work, go on.  Every wait in the kernel is bounded: on
// expiry the waiter records a status and raises a sticky abort flag that all
// other waits poll, and the kernel returns with an error code.
//
// Replaces the worker/scheduler loops of the reference runtime
// (include/mirage/persistent_kernel/persistent_kernel.cuh:693-1854) and its
// task kernels (tasks/blackwell/*.cuh, tasks/ampere/*.cuh, tasks/hopper/rmsnorm_hopper.cuh).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mk_types.h"

// This file is compiled three times into one library (see the wrappers mk_kernel_tp.cu and
// mk_kernel_hier.cu): the persistent kernel runs every op body once per layer out of a cold
// instruction cache, and code that is merely present in an op (a branch for another
// configuration, the registers it pins) measurably slows the batch-1 step down.  So the
// single-GPU kernels carry no tensor-parallel exchange code (+2.8 % when present) and only the
// kernels launched in thread-block clusters carry the hierarchical grid barrier (+2.0 %).
//   MK_VARIANT        inner namespace of this compilation: base | tp | hier
//   MK_WITH_XCHG      1: linear epilogues can push to / input staging can gather from the ranks' exchange regions
//   MK_HIER_BARRIER   1: cluster-first grid barrier (the kernel must be launched with a cluster dimension)
//   MK_WITH_MOE       1: the mixture-of-experts ops (routing, per-expert row-owner linears, weighted combine)
#ifndef MK_VARIANT
#define MK_VARIANT base
#endif
#ifndef MK_WITH_XCHG
#define MK_WITH_XCHG 0
#endif
#ifndef MK_HIER_BARRIER
#define MK_HIER_BARRIER 0
#endif
#ifndef MK_WITH_MOE
#define MK_WITH_MOE 0
#endif
#if MK_WITH_XCHG
#define MK_XF(op, f) ((op).flags & (f))
#else
#define MK_XF(op, f) 0
#endif

namespace mk {
namespace MK_VARIANT {

// ------------------------------------------------------------------------------------
// PTX helpers
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// 2-D tiled TMA load into this CTA only: box {64 k-elements, 128 rows} at (x = k, y = row).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// The same with an L2 eviction policy (from createpolicy) attached to the lines it reads.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// barrier counter and abort flag (adjacent words) in one load
__device__ __forceinline__ uint2 ld_bar_pair(const unsigned* p) {
  uint2 v;
  asm volatile("ld.acquire.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ------------------------------------------------------------------------------------
// per-thread context
// ------------------------------------------------------------------------------------
struct Ctx {
  const KParams& p;
  uint8_t* smem;
  uint32_t smem_addr;
  unsigned epoch;     // grid barriers passed
  unsigned cons_idx;  // weight stages consumed
  unsigned xphase;    // per stage: parity of the next activation-box phase (only some ops use the boxes)
  bool arrived;       // this CTA has already arrived at the coming grid barrier
  int attn_iter;      // iteration whose attention metadata is cached in shared memory
  uint32_t tmem;      // base address of the CTA's tensor-memory columns
  bool has_tmem;
  unsigned done_phase;  // phases of the accumulator-ready mbarrier consumed so far
  int tid, lane, warp;
  int iter, cur_op;
  unsigned long long* dbg;  // inner-phase stamps of the traced op (thread 0), or null
  unsigned long long* pr;   // this op's trace record, or null
  bool dead;                // abort flag seen at the op's barrier (CTA-uniform)
  unsigned ar_seq;          // cross-rank exchanges (allreduce pushes) executed so far in this launch
  unsigned lin_seq;         // linear ops whose barrier has been passed in this launch
#if MK_HIER_BARRIER
  unsigned nbar;            // grid barriers waited for in this launch (phase of the cluster mbarriers)
  uint32_t cl_rank, cl_size;  // this CTA's rank in its thread-block cluster, CTAs per cluster
#endif
  __device__ Ctx(const KParams& p_) : p(p_) {}
  __device__ uint32_t full_bar(int s) const { return smem_addr + p.bar_off + 8 * s; }
  __device__ uint32_t empty_bar(int s) const { return smem_addr + p.bar_off + 8 * (p.num_stages + s); }
  __device__ uint32_t xfull_bar(int s) const { return smem_addr + p.bar_off + 8 * (2 * p.num_stages + s); }
  __device__ volatile int* flags() const { return (volatile int*)(smem + p.bar_off + 24 * p.num_stages); }
  // behind the flags: the accumulator-ready mbarrier of the tcgen05 path and the word tcgen05.alloc writes
  __device__ uint32_t done_bar() const { return smem_addr + p.bar_off + 24 * p.num_stages + 64; }
  __device__ uint32_t tmem_slot() const { return smem_addr + p.bar_off + 24 * p.num_stages + 72; }
  // hierarchical grid barrier: arrivals of the cluster (used in its first CTA), release from the first CTA, its abort word
  __device__ uint32_t cl_arrive_bar() const { return smem_addr + p.bar_off + 24 * p.num_stages + 80; }
  __device__ uint32_t cl_open_bar() const { return smem_addr + p.bar_off + 24 * p.num_stages + 88; }
  __device__ uint32_t cl_dead_word() const { return smem_addr + p.bar_off + 24 * p.num_stages + 96; }
  __device__ float* sums() const { return (float*)(smem + p.sums_off); }
  __device__ float* red() const { return (float*)(smem + p.red_off); }  // small scratch: reductions, lengths
};
// flags(): [0] go word written by consumers, read by the producer
//          [1] stages issued by the producer   [2] broadcast slot   [3] dead flag of the op
//          [4] linear ops whose barrier the consumers have passed   [5] activation stages issued

#define MK_STAMP(c, k)                                             \
  do {                                                            \
    if ((c).dbg != nullptr && (c).tid == 0) (c).dbg[k] = globaltimer(); \
  } while (0)

__device__ __noinline__ void raise_abort(const Ctx& c, int code, int d0, int d1) {
  if (atomicCAS(c.p.abort_flag, 0, 1) == 0) {
    c.p.status[0] = code;
    c.p.status[1] = blockIdx.x;
    c.p.status[2] = c.cur_op;
    c.p.status[3] = c.iter;
    c.p.status[4] = d0;
    c.p.status[5] = d1;
    c.p.status[6] = threadIdx.x;
    __threadfence();
  }
}
__device__ __forceinline__ bool aborted(const Ctx& c) { return *(volatile int*)c.p.abort_flag != 0; }

// Bounded wait on an mbarrier phase.  Returns false after raising the abort flag.
// The clock is only consulted every few thousand failed polls: reading %globaltimer
// is slow enough to throttle the weight stream if it sits on the per-tile path.
// Time limits are tiered so that the record names the root cause: a wait on another GPU gives
// up after timeout_ns, waits on other CTAs or on the producer after twice that, the producers'
// own waits (on the consumers) after four times.
__device__ __noinline__ bool mbar_wait_slow(const Ctx& c, uint32_t bar, uint32_t parity, int code) {
  unsigned long long t0 = 0;
  unsigned polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (((++polls) & 4095u) == 0) {
      if (aborted(c)) return false;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > c.p.timeout_ns * (code == ST_TIMEOUT_EMPTY ? 4ull : 2ull)) {
        raise_abort(c, code, (int)bar, (int)parity);
        return false;
      }
    }
  }
}
// Fast path: a few hundred polls without touching the clock; then the bounded slow path.
__device__ __forceinline__ bool mbar_wait(const Ctx& c, uint32_t bar, uint32_t parity, int code) {
#pragma unroll 1
  for (int i = 0; i < 256; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(c, bar, parity, code);
}

// Grid-wide barrier of the consumer warps.  The counter only grows within a launch: barrier
// number e is passed when it reaches e * (arrivals per barrier), compared modulo 2^32 so
// that a long launch may wrap it.
//
// Two shapes, chosen by the host per launch (KParams::cluster):
//  * flat (cluster = 1): every CTA adds 1 to the counter in L2 and polls it.
//  * hierarchical (cluster = 2 or 4, the kernel is launched in thread-block clusters): the CTAs
//    of a cluster first meet on an mbarrier in the shared memory of the cluster's first CTA
//    (remote arrive over distributed shared memory, release at cluster scope); that CTA alone
//    adds 1 to the global counter, polls it, and then opens an mbarrier in each of its peers'
//    shared memory.  The global line sees gridDim.x / cluster arrivals and pollers instead of
//    gridDim.x.  (The reference's Fleet runtime counts arrivals per XCD before one global release
//    per XCD, persistent_kernel.cuh:1214-1275; this is the same idea on Blackwell's clusters.)
//
// The arrival half on its own: an op that has loads to issue which do not depend on other
// CTAs arrives first and issues them while the others catch up.
#if MK_HIER_BARRIER
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on an mbarrier that CTAs of the same cluster arrive on.
__device__ __noinline__ bool cluster_bar_wait(const Ctx& c, uint32_t bar, uint32_t parity) {
  unsigned long long t0 = 0;
  unsigned polls = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (((++polls) & 1023u) == 0) {
      if (aborted(c)) return false;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2 * c.p.timeout_ns) {
        raise_abort(c, ST_TIMEOUT_GRID, (int)c.epoch, -(int)c.cl_rank - 1);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void grid_arrive(Ctx& c) {
  consumer_sync();
  c.epoch += 1;
  c.arrived = true;
  if (c.tid == 0) {
    // arrive with a release: nothing comes back, polling can start at once
    if (c.cl_size == 1) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.p.grid_bar) : "memory");
    else mbar_arrive_cluster(cluster_map(c.cl_arrive_bar(), 0));
  }
}
// The waiting half.  Inlined where values loaded ahead of the barrier must stay in registers
// (a call would spill them, and a spill waits for the load).
__device__ __forceinline__ void grid_wait(Ctx& c) {
  c.arrived = false;
  if (c.tid == 0) {
    bool dead = false;
    if (c.cl_rank == 0) {
      if (c.cl_size > 1) {
        // the cluster is complete: one arrival for all of it (the release is cumulative over what
        // the peers published to this thread through the mbarrier)
        if (cluster_bar_wait(c, c.cl_arrive_bar(), c.nbar & 1u))
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.p.grid_bar) : "memory");
        else
          dead = true;
      }
      const unsigned target = c.epoch * (gridDim.x / c.cl_size);
      unsigned long long t0 = 0;
      unsigned spins = 0;
      // the abort flag is the word behind the counter: one 8-byte load polls both
      while (!dead) {
        const uint2 v = ld_bar_pair(c.p.grid_bar);
        if (v.y != 0u) {
          dead = true;
          break;
        }
        if ((int)(v.x - target) >= 0) break;
        if (((++spins) & 1023u) == 0) {
          const unsigned long long now = globaltimer();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > 2 * c.p.timeout_ns) {
            raise_abort(c, ST_TIMEOUT_GRID, (int)c.epoch, (int)ld_acquire_u32(c.p.grid_bar));
            dead = true;
            break;
          }
        }
      }
      for (uint32_t r = 1; r < c.cl_size; ++r) {
        asm volatile("st.relaxed.cluster.shared::cluster.u32 [%0], %1;" ::"r"(cluster_map(c.cl_dead_word(), r)), "r"(dead ? 1u : 0u) : "memory");
        mbar_arrive_cluster(cluster_map(c.cl_open_bar(), r));
      }
    } else {
      if (!cluster_bar_wait(c, c.cl_open_bar(), c.nbar & 1u)) dead = true;
      else dead = *reinterpret_cast<volatile uint32_t*>(c.smem + c.p.bar_off + 24 * c.p.num_stages + 96) != 0u;
    }
    c.flags()[3] = dead ? 1 : 0;
  }
  c.nbar += 1;
  consumer_sync();
}
#else
__device__ __forceinline__ void grid_arrive(Ctx& c) {
  consumer_sync();
  c.epoch += 1;
  c.arrived = true;
  // arrive with a release reduction: nothing comes back, polling can start at once
  if (c.tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.p.grid_bar) : "memory");
}
// The waiting half.  Inlined where values loaded ahead of the barrier must stay in registers
// (a call would spill them, and a spill waits for the load).
__device__ __forceinline__ void grid_wait(Ctx& c) {
  c.arrived = false;
  if (c.tid == 0) {
    const unsigned target = c.epoch * gridDim.x;
    unsigned long long t0 = 0;
    unsigned spins = 0;
    // the abort flag is the word behind the counter: one 8-byte load polls both
    bool dead = false;
    while (true) {
      const uint2 v = ld_bar_pair(c.p.grid_bar);
      if (v.y != 0u) {
        dead = true;
        break;
      }
      if ((int)(v.x - target) >= 0) break;
      if (((++spins) & 1023u) == 0) {
        const unsigned long long now = globaltimer();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > 2 * c.p.timeout_ns) {
          raise_abort(c, ST_TIMEOUT_GRID, (int)c.epoch, (int)ld_acquire_u32(c.p.grid_bar));
          dead = true;
          break;
        }
      }
    }
    c.flags()[3] = dead ? 1 : 0;
  }
  consumer_sync();
}
#endif  // MK_HIER_BARRIER
__device__ __noinline__ void grid_sync(Ctx& c) {
  if (!c.arrived) grid_arrive(c);
  grid_wait(c);
}

// Every op calls this once, after whatever it can fetch ahead of its dependencies:
// the grid barrier (if the op has one) and the CTA-uniform abort check.  Returns
// true when the abort flag is up and the op body must be skipped.
__device__ __forceinline__ bool op_barrier(Ctx& c, const OpDesc& op) {
  if (op.flags & F_SYNC_BEFORE) {
    grid_sync(c);
  } else {
    if (c.tid == 0) c.flags()[3] = aborted(c) ? 1 : 0;
    consumer_sync();
  }
  if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
  c.dead = c.flags()[3] != 0;
  return c.dead;
}

// Sum over the 256 consumer threads; every thread gets the result.
__device__ __forceinline__ float block_sum(Ctx& c, float v) {
  float* r = c.red();  // scratch behind the 128x4 accumulator block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (c.lane == 0) r[c.warp] = v;
  consumer_sync();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kNumConsumerWarps; ++i) s += r[i];
  consumer_sync();
  return s;
}

// ------------------------------------------------------------------------------------
// tensor-parallel exchange over NVLink peer memory (the two allreduces of a layer)
// ------------------------------------------------------------------------------------
// The reference's allreduce is an NVSHMEM put-with-signal allgather followed by a local
// reduction task (src/kernel/task_register.cc:1606-1687, tasks/ampere/reduction.cuh:139-166).
// Here every rank stores its fp32 partial sums straight into EVERY rank's exchange region
// (its own included) with plain stores over NVLink, as 8-byte words {value, exchange number}:
// a word that carries the awaited number has arrived, so no fence, flag or second round trip
// is needed, and a reader simply adds the ranks' words up in rank order in fp32 (identical
// on every rank) and rounds once to bf16.  Data always lands in the reader's own memory; no
// bulk or tensor copy ever touches a peer's memory.  The halves of a region alternate between
// consecutive exchanges: a rank can only push exchange s+2 after it has read all of s+1 from
// every peer, which those peers push after their last read of s.
__device__ __forceinline__ uint4 ld_sys_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_sys_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_v2(uint2* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_sys_v4(uint4* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// one value of exchange `seq` into every rank's region
__device__ __forceinline__ void xchg_push1(const KParams& p, unsigned seq, int tok, int col, float v) {
  const size_t w = xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, p.rank, tok, col);
#pragma unroll 1
  for (int r = 0; r < p.world; ++r) st_sys_v2(reinterpret_cast<uint2*>(p.xchg[r]) + w, __float_as_uint(v), seq);
}
// A word of a rank that is not there yet: poll it (bounded).  Returns false after raising the abort flag.
__device__ __noinline__ bool xchg_wait_word(const Ctx& c, const uint2* w, unsigned seq, int src) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    if (xchg_arrived(ld_sys_v2(w).y, seq)) return true;
    if (((++spins) & 63u) == 0) {
      if (aborted(c)) return false;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > c.p.timeout_ns) {
        raise_abort(c, ST_TIMEOUT_RANK, src, (int)seq);
        return false;
      }
    }
  }
}
// 8 consecutive columns (col a multiple of 8) of token row `tok`: the sum over ranks as bf16 x 8
__device__ __noinline__ uint4 xchg_gather8(const Ctx& c, unsigned seq, int tok, int col) {
  const KParams& p = c.p;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 1
  for (int r = 0; r < p.world; ++r) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint2*>(p.xchg[p.rank]) +
                                                      xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, r, tok, col));
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = ld_sys_v4(src + i);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!xchg_arrived(q[i].y, seq) || !xchg_arrived(q[i].w, seq)) {
        const uint2* w2 = reinterpret_cast<const uint2*>(src + i);
        if (!xchg_wait_word(c, w2, seq, r) || !xchg_wait_word(c, w2 + 1, seq, r)) return make_uint4(0, 0, 0, 0);
        q[i] = ld_sys_v4(src + i);
      }
      acc[2 * i] += __uint_as_float(q[i].x);
      acc[2 * i + 1] += __uint_as_float(q[i].z);
    }
  }
  return pack8(acc);
}
// one column: the bf16-rounded sum over ranks, as a float
__device__ __noinline__ float xchg_gather1(const Ctx& c, unsigned seq, int tok, int col) {
  const KParams& p = c.p;
  float acc = 0.f;
#pragma unroll 1
  for (int r = 0; r < p.world; ++r) {
    const uint2* w = reinterpret_cast<const uint2*>(p.xchg[p.rank]) + xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, r, tok, col);
    uint2 q = ld_sys_v2(w);
    if (!xchg_arrived(q.y, seq)) {
      if (!xchg_wait_word(c, w, seq, r)) return 0.f;
      q = ld_sys_v2(w);
    }
    acc += __uint_as_float(q.x);
  }
  return rbf(acc);
}
// number of the latest exchange (the one gathering ops read) and of the one a pushing linear writes
__device__ __forceinline__ unsigned xchg_cur(const Ctx& c) { return xchg_seq(c.p.xchg_seq_base, c.ar_seq); }
__device__ __forceinline__ unsigned xchg_next(const Ctx& c) { return xchg_seq(c.p.xchg_seq_base, c.ar_seq + 1u); }

// ------------------------------------------------------------------------------------
// Tagged activations between the ops of the row-owner path.  A producer stores every pair of adjacent
// bf16 outputs as one 8-byte word {pair, tag}; 8-byte stores are single-copy atomic, so a word that
// carries the awaited tag carries its data: the consumer needs no grid barrier, no fence and no second
// round trip, it simply polls the words it is going to read anyway.  Eight columns are four words,
// read as two 16-byte loads.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_gpu_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_gpu_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_gpu_v2(uint2* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ bool ll_ok(const uint4& a, const uint4& b, unsigned tag) {
  return a.y == tag && a.w == tag && b.y == tag && b.w == tag;
}
// Eight columns whose words have not all arrived: poll them (bounded).  Zeros after the abort flag went up.
__device__ __noinline__ uint4 ll_wait8(const Ctx& c, const uint4* src, unsigned tag) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    const uint4 a = ld_gpu_v4(src), b = ld_gpu_v4(src + 1);
    if (ll_ok(a, b, tag)) return make_uint4(a.x, a.z, b.x, b.z);
    if (((++spins) & 63u) == 0) {
      if (aborted(c)) return make_uint4(0, 0, 0, 0);
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2 * c.p.timeout_ns) {
        raise_abort(c, ST_TIMEOUT_DATA, (int)tag, (int)a.y);
        return make_uint4(0, 0, 0, 0);
      }
    }
  }
}
__device__ __forceinline__ uint4 ll_take8(const Ctx& c, const uint4* src, const uint4& a, const uint4& b, unsigned tag) {
  return ll_ok(a, b, tag) ? make_uint4(a.x, a.z, b.x, b.z) : ll_wait8(c, src, tag);
}
// eight columns from column `col` (a multiple of 8) of the row that starts at word `row`
__device__ __forceinline__ uint4 ll_gather8(const Ctx& c, const uint2* row, int col, unsigned tag) {
  const uint4* src = reinterpret_cast<const uint4*>(row + (col >> 1));
  const uint4 a = ld_gpu_v4(src), b = ld_gpu_v4(src + 1);
  return ll_take8(c, src, a, b, tag);
}
// one column, as a float
__device__ __noinline__ float ll_gather1(const Ctx& c, const uint2* row, int col, unsigned tag) {
  const uint2* w = row + (col >> 1);
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    const uint2 q = ld_gpu_v2(w);
    if (q.y == tag) return (col & 1) ? bf_hi(q.x) : bf_lo(q.x);
    if (((++spins) & 63u) == 0) {
      if (aborted(c)) return 0.f;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2 * c.p.timeout_ns) {
        raise_abort(c, ST_TIMEOUT_DATA, (int)tag, (int)q.y);
        return 0.f;
      }
    }
  }
}
__device__ __forceinline__ const uint2* ll_row(const void* base, int ld, int tok) {
  return reinterpret_cast<const uint2*>(base) + (size_t)tok * (size_t)(ld >> 1);
}
// the tag of what program op `op` stores in the current iteration
__device__ __forceinline__ unsigned ll_tag_of(const Ctx& c, int op) { return ll_tag(c.iter, c.p.num_ops, op); }

#if MK_WITH_XCHG
// Tensor parallelism, row-owner path: the reader of an exchange does not add up all of it in every CTA
// (that is `world` dependent round trips per CTA and `world` times the row in loads).  Every CTA adds up
// its own slice of the columns, in rank order in fp32 with one bf16 rounding (the same value on every
// rank), and stores it as tagged words; all CTAs then stage the row from those words like any other
// tagged input: two round trips whatever the number of ranks.
__device__ __noinline__ void xchg_reduce_slice(Ctx& c, const OpDesc& op, int T) {
  const KParams& p = c.p;
  const int pairs = op.k >> 1;
  const int p0 = (int)((long long)blockIdx.x * pairs / gridDim.x), p1 = (int)((long long)(blockIdx.x + 1) * pairs / gridDim.x);
  const int w = p1 - p0;
  const unsigned seq = xchg_cur(c);
  const unsigned tag = ll_tag_of(c, c.cur_op);
  uint2* dst = reinterpret_cast<uint2*>(const_cast<void*>(op.ll_in));
#pragma unroll 1
  for (int i = c.tid; i < w * T; i += kNumConsumers) {
    const int tok = i / w, pr = p0 + i % w;
    uint4 q[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < p.world)
        q[r] = ld_sys_v4(reinterpret_cast<const uint4*>(reinterpret_cast<const uint2*>(p.xchg[p.rank]) +
                                                        xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, r, tok, 2 * pr)));
    }
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < p.world) {
        if (!xchg_arrived(q[r].y, seq) || !xchg_arrived(q[r].w, seq)) {
          const uint2* w2 = reinterpret_cast<const uint2*>(p.xchg[p.rank]) + xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, r, tok, 2 * pr);
          if (!xchg_wait_word(c, w2, seq, r) || !xchg_wait_word(c, w2 + 1, seq, r)) return;
          q[r] = ld_sys_v4(reinterpret_cast<const uint4*>(w2));
        }
        a0 += __uint_as_float(q[r].x);
        a1 += __uint_as_float(q[r].z);
      }
    }
    st_gpu_v2(dst + (size_t)tok * (size_t)(op.ld_in >> 1) + pr, pack2(a0, a1), tag);
  }
}
#endif

// ------------------------------------------------------------------------------------
__device__ __noinline__ float torch_rsqrt_bf16(float var, bool dbl);

// activations -> shared memory, with the optional fused RMSNorm
// ------------------------------------------------------------------------------------
// Stages rows tok0 .. tok0+rows-1 of `in` as bf16 [rows][pitch] in the x region
// (pitch = padded K + 8 elements, so that the 8 token rows of an ldmatrix hit 8
// different banks), zero padded, followed by one 16-byte chunk of zeros that
// stands in for the rows of absent tokens.
// Stage `rows` (at most 8) token rows (tokens tok0.. of T; absent ones zero) of a K-wide
// bf16 input in shared memory, row pitch kp + 8, RMS-normalised when norm_w is given.  All
// rows are staged concurrently: the 8 consumer warps split into one group per row (8 warps
// on a single row, 1 warp per row for 5 to 8 rows), a group's warps take interleaved
// 512-byte pieces of the row and meet once to add up their sums of squares.  The loops are
// kept rolled on purpose: this runs once per op, straight from a cold instruction cache.
//
// `pre_w`: when not null, this lane's first 4 norm-weight vectors (vector index
// part * 32 + lane + 32 * wpr * i), loaded by the caller ahead of the op's barrier; rows of
// at most 4 vectors per lane then stay in registers between the two passes.
__device__ __forceinline__ int stage_warps_per_row(int rows) { return rows <= 1 ? 8 : (rows == 2 ? 4 : (rows <= 4 ? 2 : 1)); }

// sum of squares of 8 bf16 values; `torch_num`: each square rounded to bf16 first
__device__ __forceinline__ float sumsq8(const uint4& val, bool torch_num, float ss) {
  float f[8];
  unpack8(val, f);
  if (torch_num) {
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += rbf(f[i] * f[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  return ss;
}
// 8 values scaled by r and the norm weight: w * bf16(x * r), or x * (r * w) in fp32
__device__ __forceinline__ uint4 scale8(const uint4& val, const uint4& wvec, float r, bool torch_num) {
  float f[8], w[8];
  unpack8(val, f);
  unpack8(wvec, w);
  if (torch_num) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = w[i] * rbf(f[i] * r);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * (r * w[i]);
  }
  return pack8(f);
}

// The scaling factor of a row from the sums of squares its warps left in red[].
__device__ __forceinline__ float row_rms_scale(const float* red, int first, int wpr, int K, bool torch_num) {
  float ss = 0.f;
  for (int q = 0; q < wpr; ++q) ss += red[first + q];
  // reference PyTorch RMSNorm: bf16 mean of bf16 squares, bf16 rsqrt, two bf16 products
  // (a one-element bf16 rsqrt on the CPU is 1 / bf16(sqrt(x)) rounded again)
  return torch_num ? torch_rsqrt_bf16(rbf(ss / (float)K), true) : rsqrtf(ss / (float)K + 1e-6f);
}

// A normalised row of at most NV vectors per lane, kept in registers between the sum of
// squares and the scaling; the norm weights were loaded ahead of the op's barrier.
template <int NV>
__device__ __forceinline__ void stage_row_regs(Ctx& c, const uint4* src, uint4* dst, const uint4* pre_w, int K, int nvec,
                                               int v0, int vstep, bool active, bool valid, int red_first, int wpr,
                                               bool gather, int tok, uint4* sum_row) {
  const int kvec = K >> 3;
  const bool torch_num = c.p.numerics == NUM_TORCH;
  float* red = c.red();
  uint4 raw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = v0 + vstep * i;
    raw[i] = (valid && v < kvec && !gather) ? __ldcg(src + v) : make_uint4(0, 0, 0, 0);
  }
  if (gather) {  // (kept apart from the plain loads above: a call between them would serialise them)
#if MK_WITH_XCHG
    if constexpr (NV == 2) {
      // both vectors of a rank in flight together, the ranks one after the other: `world` round trips, not 2 x world
      const KParams& p = c.p;
      const unsigned seq = xchg_cur(c);
      float acc[2][8];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
#pragma unroll 1
      for (int r = 0; r < p.world; ++r) {
        uint4 q[2][4];
        const uint4* src4[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int v = min(v0 + vstep * i, kvec - 1);
          src4[i] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint2*>(p.xchg[p.rank]) +
                                                   xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, r, tok, v * 8));
#pragma unroll
          for (int k = 0; k < 4; ++k) q[i][k] = (valid && v0 + vstep * i < kvec) ? ld_sys_v4(src4[i] + k) : make_uint4(0u, seq, 0u, seq);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (!(valid && v0 + vstep * i < kvec)) continue;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (!xchg_arrived(q[i][k].y, seq) || !xchg_arrived(q[i][k].w, seq)) {
              const uint2* w2 = reinterpret_cast<const uint2*>(src4[i] + k);
              if (xchg_wait_word(c, w2, seq, r) && xchg_wait_word(c, w2 + 1, seq, r)) q[i][k] = ld_sys_v4(src4[i] + k);
            }
            acc[i][2 * k] += __uint_as_float(q[i][k].x);
            acc[i][2 * k + 1] += __uint_as_float(q[i][k].z);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int v = v0 + vstep * i;
        if (valid && v < kvec) {
          raw[i] = pack8(acc[i]);
          if (sum_row != nullptr) sum_row[v] = raw[i];  // the reduced row, for a later reader of the tensor itself (a residual)
        }
      }
    } else
#endif
    {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = v0 + vstep * i;
        if (valid && v < kvec) {
          raw[i] = xchg_gather8(c, xchg_cur(c), tok, v * 8);
          if (sum_row != nullptr) sum_row[v] = raw[i];
        }
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) ss = sumsq8(raw[i], torch_num, ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (c.lane == 0) red[c.warp] = ss;
  consumer_sync();
  if (active) {
    const float r = row_rms_scale(red, red_first, wpr, K, torch_num);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = v0 + vstep * i;
      if (v < nvec) dst[v] = scale8(raw[i], pre_w[i], r, torch_num);
    }
  }
  consumer_sync();
}

// `gather`: the rows are not read from `in` but summed over the ranks' slots of the latest exchange.
__device__ __noinline__ void stage_x(Ctx& c, const void* in, int ld_in, int K, int kp, const void* norm_w, int tok0,
                                     int rows, int T, const uint4* pre_w, bool gather = false, void* sums_out = nullptr) {
  if (!MK_WITH_XCHG) gather = false;  // (compiled out of the single-GPU build)
  uint4* xs = reinterpret_cast<uint4*>(c.smem + c.p.x_off);
  const int pitch = (kp >> 3) + 1;  // uint4 per row
  const int nvec = kp >> 3, kvec = K >> 3;
  const bool torch_num = c.p.numerics == NUM_TORCH;
  const uint4* wv = reinterpret_cast<const uint4*>(norm_w);
  const int wpr = stage_warps_per_row(rows);
  const int tb = c.warp / wpr, part = c.warp % wpr;
  const bool active = tb < rows;
  const bool valid = active && tok0 + tb < T;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(in) + (size_t)(tok0 + tb) * ld_in);
  uint4* dst = xs + tb * pitch;
  float* red = c.red();
  const int v0 = part * 32 + c.lane, vstep = 32 * wpr;
  if (c.tid == 0) xs[rows * pitch] = make_uint4(0, 0, 0, 0);  // the chunk absent tokens point at
  if (active && part == 0 && c.lane == 0) dst[nvec] = make_uint4(0, 0, 0, 0);  // the row's padding vector
  if (wv != nullptr && pre_w != nullptr && nvec <= 4 * vstep) {
    uint4* sum_row = (gather && sums_out != nullptr && valid) ? reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(sums_out) + (size_t)(tok0 + tb) * ld_in)
                                                              : nullptr;
    if (nvec <= 2 * vstep) stage_row_regs<2>(c, src, dst, pre_w, K, nvec, v0, vstep, active, valid, tb * wpr, wpr, gather, tok0 + tb, sum_row);
    else stage_row_regs<4>(c, src, dst, pre_w, K, nvec, v0, vstep, active, valid, tb * wpr, wpr, gather, tok0 + tb, sum_row);
    return;
  }
  float ss = 0.f;
  if (active) {
    // four loads in flight at a time (a store to shared memory between two loads would
    // order them: the compiler cannot tell the two address spaces apart here)
#pragma unroll 1
    for (int vb = v0; vb < nvec; vb += 4 * vstep) {
      uint4 val[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = vb + i * vstep;
        val[i] = (valid && v < kvec && !gather) ? __ldcg(src + v) : make_uint4(0, 0, 0, 0);
      }
      if (gather) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int v = vb + i * vstep;
          if (valid && v < kvec) val[i] = xchg_gather8(c, xchg_cur(c), tok0 + tb, v * 8);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = vb + i * vstep;
        if (v < nvec) {
          dst[v] = val[i];
          if (wv != nullptr) ss = sumsq8(val[i], torch_num, ss);
        }
      }
    }
  }
  if (wv != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (c.lane == 0) red[c.warp] = ss;
    consumer_sync();
    if (active) {
      const float r = row_rms_scale(red, tb * wpr, wpr, K, torch_num);
#pragma unroll 2
      for (int v = v0; v < kvec; v += vstep)  // a lane re-reads only what it wrote itself
        dst[v] = scale8(dst[v], __ldg(wv + v), r, torch_num);
    }
  }
  consumer_sync();
}

// Staging for a row-owner linear WITHOUT a fused norm (one or two token rows, at most 24 stages
// of 512 k): warp w multiplies only the w-th 64-wide slice of every stage, so it stages exactly
// those slices of the row itself, all in one round of loads, and needs no CTA-wide sync before
// its first tile.  Lane l takes the 16-byte chunk (l & 7) of the slices of stages (l >> 3) + 4 i.
// (The same scheme with the norm fused in was 0.36 ms per step SLOWER: its unrolled scaling code
// is several KB that every op would run once, out of a cold instruction cache.)
__device__ __noinline__ void stage_x_rows(Ctx& c, const void* in, int ld_in, int K, int kp, int tok0, int rows, int T) {
  constexpr int kMaxV = 6;  // 24 stages / 4 per round
  uint4* xs = reinterpret_cast<uint4*>(c.smem + c.p.x_off);
  const int pitch = (kp >> 3) + 1;  // uint4 per row
  const int v0 = ((c.lane >> 3) * kRowsStageK + c.warp * 64 + (c.lane & 7) * 8) >> 3;  // vector of the first round
  constexpr int vstep = 4 * kRowsStageK / 8;                                           // vectors per round
  const int kvec = K >> 3, nvec = kp >> 3;
  if (c.lane == 0) xs[rows * pitch] = make_uint4(0, 0, 0, 0);  // the chunk absent tokens point at (every warp writes the same zeros)
#pragma unroll 1
  for (int t = 0; t < rows; ++t) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(in) + (size_t)(tok0 + t) * ld_in);
    const bool live = tok0 + t < T;
    uint4 raw[kMaxV];
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = v0 + i * vstep;
      raw[i] = (live && v < kvec) ? __ldcg(src + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = v0 + i * vstep;
      if (v < nvec) xs[t * pitch + v] = raw[i];
    }
  }
  __syncwarp();
}

// The same two stagings for an input that arrives as tagged words (no barrier stands before the op):
// every lane first issues all its loads, then polls whatever has not arrived.  They are separate
// functions on purpose: folded into the plain ones above they slowed those down by 8 % of a step
// (registers and stack of code that runs once per op).
template <int NV>
__device__ __forceinline__ void stage_ll_regs(Ctx& c, const uint4* ll, uint4* dst, const uint4* pre_w, const uint4* wv, int K,
                                              int nvec, int v0, int vstep, bool active, bool valid, int red_first, int wpr,
                                              unsigned tag) {
  const int kvec = K >> 3;
  const bool torch_num = c.p.numerics == NUM_TORCH;
  float* red = c.red();
  uint4 qa[NV], qb[NV], raw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = v0 + vstep * i;
    const bool ok = valid && v < kvec;
    qa[i] = ok ? ld_gpu_v4(ll + 2 * v) : make_uint4(0, 0, 0, 0);
    qb[i] = ok ? ld_gpu_v4(ll + 2 * v + 1) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = v0 + vstep * i;
    raw[i] = (valid && v < kvec) ? ll_take8(c, ll + 2 * v, qa[i], qb[i], tag) : make_uint4(0, 0, 0, 0);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) ss = sumsq8(raw[i], torch_num, ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (c.lane == 0) red[c.warp] = ss;
  consumer_sync();
  if (active) {
    const float r = row_rms_scale(red, red_first, wpr, K, torch_num);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = v0 + vstep * i;
      if (v < nvec) dst[v] = scale8(raw[i], pre_w != nullptr ? pre_w[i] : (v < kvec ? __ldg(wv + v) : make_uint4(0, 0, 0, 0)), r, torch_num);
    }
  }
  consumer_sync();
}
// fused norm; the host only plans it for rows of at most four vectors per lane
__device__ __noinline__ void stage_x_ll(Ctx& c, const void* ll_in, int ld_in, int K, int kp, const void* norm_w, int tok0,
                                        int rows, int T, const uint4* pre_w, unsigned tag) {
  uint4* xs = reinterpret_cast<uint4*>(c.smem + c.p.x_off);
  const int pitch = (kp >> 3) + 1;
  const int nvec = kp >> 3;
  const int wpr = stage_warps_per_row(rows);
  const int tb = c.warp / wpr, part = c.warp % wpr;
  const bool active = tb < rows;
  const bool valid = active && tok0 + tb < T;
  const uint4* ll = reinterpret_cast<const uint4*>(ll_row(ll_in, ld_in, valid ? tok0 + tb : 0));
  uint4* dst = xs + tb * pitch;
  const int v0 = part * 32 + c.lane, vstep = 32 * wpr;
  if (c.tid == 0) xs[rows * pitch] = make_uint4(0, 0, 0, 0);
  if (active && part == 0 && c.lane == 0) dst[nvec] = make_uint4(0, 0, 0, 0);
  const uint4* wv = reinterpret_cast<const uint4*>(norm_w);
  if (nvec <= 2 * vstep) stage_ll_regs<2>(c, ll, dst, pre_w, wv, K, nvec, v0, vstep, active, valid, tb * wpr, wpr, tag);
  else stage_ll_regs<4>(c, ll, dst, pre_w, wv, K, nvec, v0, vstep, active, valid, tb * wpr, wpr, tag);
}
// no norm: every warp stages the k slices it multiplies (see stage_x_rows)
__device__ __noinline__ void stage_rows_ll(Ctx& c, const void* ll_in, int ld_in, int K, int kp, int tok0, int rows, int T, unsigned tag) {
  constexpr int kMaxV = 6;
  uint4* xs = reinterpret_cast<uint4*>(c.smem + c.p.x_off);
  const int pitch = (kp >> 3) + 1;
  const int v0 = ((c.lane >> 3) * kRowsStageK + c.warp * 64 + (c.lane & 7) * 8) >> 3;
  constexpr int vstep = 4 * kRowsStageK / 8;
  const int kvec = K >> 3, nvec = kp >> 3;
  if (c.lane == 0) xs[rows * pitch] = make_uint4(0, 0, 0, 0);
#pragma unroll 1
  for (int t = 0; t < rows; ++t) {
    const bool live = tok0 + t < T;
    const uint4* ll = reinterpret_cast<const uint4*>(ll_row(ll_in, ld_in, live ? tok0 + t : 0));
    uint4 qa[kMaxV], qb[kMaxV];
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = v0 + i * vstep;
      const bool ok = live && v < kvec;
      qa[i] = ok ? ld_gpu_v4(ll + 2 * v) : make_uint4(0, 0, 0, 0);
      qb[i] = ok ? ld_gpu_v4(ll + 2 * v + 1) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int v = v0 + i * vstep;
      if (v < nvec) xs[t * pitch + v] = (live && v < kvec) ? ll_take8(c, ll + 2 * v, qa[i], qb[i], tag) : make_uint4(0, 0, 0, 0);
    }
  }
  __syncwarp();
}

// ------------------------------------------------------------------------------------
// linear layer: weight tiles from the TMA ring x activations from shared memory on the
// warp-level tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate)
// ------------------------------------------------------------------------------------
// Each of the 8 consumer warps owns 16 of a tile's 128 weight rows (the A operand, read
// with ldmatrix from the 128-byte-swizzled stage); up to 8 tokens form the N dimension
// (the B operand, token rows read with ldmatrix from the staged activations).  Every
// (row, token) sum lives in exactly one thread, so a run of tiles ends without any
// cross-lane reduction.
struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ ArgBest arg_better(ArgBest a, ArgBest b) {
  // larger value wins; ties go to the lower index
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgBest warp_argmax(ArgBest a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = arg_better(a, b);
  }
  return a;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// ntok tokens starting at tok0; sums at sums()[row * sums_stride + token]
__device__ void linear_epilogue(Ctx& c, const OpDesc& op, int blk, int tok0, int ntok, float res0) {
  const KParams& p = c.p;
  const float* red = c.sums();
  const int kRedStride = p.sums_stride;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  if (op.flags & F_SILU_MUL) {
    // rows 0..63 of the tile are gate columns, rows 64..127 the matching up columns; with F_SILU4 the
    // weight is laid out for the row-owner path instead: units of 8 rows, [4 gate | 4 up]
    const int half = op.n >> 1;
    const bool by4 = (op.flags & F_SILU4) != 0;
    if (ntok > 2 && (op.ld_out & 7) == 0 && (blk + 1) * 64 <= half) {
      // a thread takes 8 consecutive output columns of one token: lanes of a warp read different tokens
      // (no bank conflicts in the sums block) and store 16 bytes
#pragma unroll 1
      for (int u = c.tid; u < 8 * ntok; u += kNumConsumers) {
        const int tb = u % ntok, cg = u / ntok;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int idx = cg * 8 + i;
          const int row = by4 ? ((idx >> 2) << 3) + (idx & 3) : idx;
          const float g = rbf(red[row * kRedStride + tb]);  // linear output is bf16 before the activation
          const float up = rbf(red[(by4 ? row + 4 : row + 64) * kRedStride + tb]);
          v[i] = rbf(__fdividef(g, 1.0f + __expf(-g))) * up;
        }
        *reinterpret_cast<uint4*>(out + (size_t)(tok0 + tb) * op.ld_out + blk * 64 + cg * 8) = pack8(v);
      }
      return;
    }
#pragma unroll 1
    for (int e = c.tid; e < 64 * ntok; e += kNumConsumers) {
      const int idx = e & 63, tb = e >> 6;
      const int col = blk * 64 + idx;
      const int row = by4 ? ((idx >> 2) << 3) + (idx & 3) : idx;
      const int urow = by4 ? row + 4 : row + 64;
      if (col < half) {
        const float g = rbf(red[row * kRedStride + tb]);  // linear output is bf16 before the activation
        const float u = rbf(red[urow * kRedStride + tb]);
        const float s = rbf(__fdividef(g, 1.0f + __expf(-g)));
        out[(size_t)(tok0 + tb) * op.ld_out + col] = __float2bfloat16_rn(s * u);
      }
    }
    return;
  }
  const bool with_res = (op.flags & F_RESIDUAL) && (!(op.flags & F_RES_RANK0) || p.rank == 0);
  const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(op.res);
  const bool push = MK_XF(op, F_PUSH) != 0;
  // Wide batches: a thread takes 8 consecutive output columns of one token (one 16-byte residual load, one
  // 16-byte store), four such units per round with their loads issued together: one dependent 2-byte load
  // per element made the block's finisher the slowest CTA of the op by far (at 64 tokens: 32 round trips).
  // Lanes of a warp take different tokens, so the sums block is read without bank conflicts.
  // (a pushing linear stores the eight sums of a unit as four 16-byte stores {value, number, value, number} per rank)
  const bool vec = !MK_XF(op, F_GATHER_RES) && ntok > 2 && (push || (op.ld_out & 7) == 0) && (!with_res || (op.ld_res & 7) == 0) &&
                   ((blk + 1) * kTileRows <= op.n);
  if (vec) {
    const int nunits = (kTileRows / 8) * ntok;
#pragma unroll 1
    for (int u0 = c.tid; u0 < nunits; u0 += 4 * kNumConsumers) {
      uint4 rv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int u = u0 + k * kNumConsumers;
        rv[k] = make_uint4(0, 0, 0, 0);
        if (with_res && u < nunits)
          rv[k] = __ldcg(reinterpret_cast<const uint4*>(res + (size_t)(tok0 + u % ntok) * op.ld_res + blk * kTileRows + (u / ntok) * 8));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int u = u0 + k * kNumConsumers;
        if (u < nunits) {
          const int tb = u % ntok, cg = u / ntok;
          float r[8], v[8];
          unpack8(rv[k], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = red[(cg * 8 + i) * kRedStride + tb];
            if (p.numerics == NUM_TORCH && !push) v[i] = rbf(v[i]);  // (pushed sums stay fp32: rounded once, after the ranks are added up)
            v[i] += r[i];
          }
#if MK_WITH_XCHG
          if (push) {
            const unsigned seq = xchg_next(c);
            const size_t w = xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, p.rank, tok0 + tb, blk * kTileRows + cg * 8);
#pragma unroll 1
            for (int rk = 0; rk < p.world; ++rk) {
              uint4* dstw = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(p.xchg[rk]) + w);
#pragma unroll
              for (int i = 0; i < 4; ++i) st_sys_v4(dstw + i, __float_as_uint(v[2 * i]), seq, __float_as_uint(v[2 * i + 1]), seq);
            }
            continue;
          }
#endif
          *reinterpret_cast<uint4*>(out + (size_t)(tok0 + tb) * op.ld_out + blk * kTileRows + cg * 8) = pack8(v);
        }
      }
    }
  } else
#pragma unroll 1
  for (int e = c.tid; e < kTileRows * ntok; e += kNumConsumers) {
    const int row = e & 127, tb = e >> 7;
    const int tok = tok0 + tb, col = blk * kTileRows + row;
    if (col < op.n) {
      float v = red[row * kRedStride + tb];
      if (p.numerics == NUM_TORCH && !push) v = rbf(v);  // (pushed partial sums stay fp32: they are rounded once, after the ranks are added up)
      if (with_res) {
        float r;
        if (e < kNumConsumers) r = res0;
        else if (MK_XF(op, F_GATHER_RES)) r = xchg_gather1(c, xchg_cur(c), tok, col);
        else r = __bfloat162float(__ldcg(res + (size_t)tok * op.ld_res + col));
        v += r;
      }
      if (push) xchg_push1(p, xchg_next(c), tok, col, v);
      else out[(size_t)tok * op.ld_out + col] = __float2bfloat16_rn(v);
    }
  }
  if (op.flags & F_ARGMAX) {
    // one warp per token: the tile's 128 bf16 logits of the token, four per lane
#pragma unroll 1
    for (int tb = c.warp; tb < ntok; tb += kNumConsumerWarps) {
      ArgBest b;
      b.v = -INFINITY;
      b.i = 0x7fffffff;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int row = c.lane + 32 * q, col = blk * kTileRows + row;
        if (col < op.n) {
          ArgBest x;
          x.v = rbf(red[row * kRedStride + tb]);
          x.i = col;
          b = arg_better(b, x);
        }
      }
      b = warp_argmax(b);
      if (c.lane == 0) {
        op.amax_val[(size_t)(tok0 + tb) * op.amax_n + blk] = b.v;
        op.amax_idx[(size_t)(tok0 + tb) * op.amax_n + blk] = b.i;
      }
    }
  }
}

// Called by all consumers at the end of a run of tiles of one row block, after the
// per-row sums of the run were left in sums()[row * sums_stride + token].
//
// When several CTAs hold k-ranges of the block, the CTA with the block's FIRST k-range
// finishes it: that range is the tail of its own tile range, so it is the last piece to
// be computed anyway.  The others publish their partial sums with a release and move on
// without waiting for anything; the finisher waits (bounded) until they have all
// arrived, adds the pieces in CTA order and runs the epilogue.
__device__ __noinline__ void linear_finish_piece(Ctx& c, const OpDesc& op, int blk, int kt_first, int kt_last,
                                                 bool first_of_cta, int tok0, int ntok, int group, float res0) {
  const KParams& p = c.p;
  float* red = c.sums();
  const int kRedStride = p.sums_stride;
  const int nvec4 = kTileRows * kRedStride / 4;  // float4 pieces of the sums block
  consumer_sync();
  const bool whole = (kt_first == 0) && (kt_last == op.nkt - 1);
  if (!whole) {
    const unsigned total = (unsigned)op.nblk * (unsigned)op.nkt;
    const int G = (int)min(gridDim.x, total);  // CTAs that hold tiles of this op
    const int GS = gridDim.x;
    const size_t slot_elems = (size_t)kTileRows * kRedStride;
    const int c_first = tile_owner((unsigned)blk * op.nkt, total, G);
    const int c_last = tile_owner((unsigned)blk * op.nkt + op.nkt - 1, total, G);
    unsigned* cnt = p.piece_count + (size_t)group * p.piece_stride + blk;
    float4* red4 = reinterpret_cast<float4*>(red);
    if ((int)blockIdx.x != c_first) {
      float4* mine = reinterpret_cast<float4*>(
          p.partial + (((size_t)group * GS + blockIdx.x) * 2 + (first_of_cta ? 0 : 1)) * slot_elems);
#pragma unroll 1
      for (int i = c.tid; i < nvec4; i += kNumConsumers) mine[i] = red4[i];
      consumer_sync();  // thread 0's release covers what the CTA wrote before this sync
      if (c.tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
      return;
    }
    const unsigned want = (unsigned)(c_last - c_first);
    if (c.tid == 0) {
      unsigned long long t0 = 0;
      unsigned spins = 0;
      while (ld_acquire_u32(cnt) < want) {
        if (((++spins) & 1023u) == 0) {
          if (aborted(c)) break;
          const unsigned long long now = globaltimer();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > 2 * c.p.timeout_ns) {
            raise_abort(c, ST_TIMEOUT_PEER, blk, (int)ld_acquire_u32(cnt));
            break;
          }
        }
      }
      *cnt = 0u;
    }
    consumer_sync();
    __threadfence();
    // all pieces' loads go out together: one L2 round trip instead of one per piece
#pragma unroll 2
    for (int i = c.tid; i < nvec4; i += kNumConsumers) {
      float4 acc = red4[i];
#pragma unroll 1
      for (int c0 = c_first + 1; c0 <= c_last; c0 += 4) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c0 + u;
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (cc <= c_last) {
            const bool first = (tile_begin(cc, total, G) / op.nkt) == blk;
            const float4* src = reinterpret_cast<const float4*>(
                p.partial + (((size_t)group * GS + cc) * 2 + (first ? 0 : 1)) * slot_elems);
            v[u] = __ldcg(src + i);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc.x += v[u].x;
          acc.y += v[u].y;
          acc.z += v[u].z;
          acc.w += v[u].w;
        }
      }
      red4[i] = acc;
    }
    consumer_sync();
  }
  linear_epilogue(c, op, blk, tok0, ntok, res0);
  consumer_sync();
}

// Tokens one pass of a linear op covers (aux3, fixed by the host from the shared-memory
// budget) and the passes its weight stream makes for T active tokens.
__device__ __forceinline__ int linear_passes(const OpDesc& op, int T) { return (T + op.aux3 - 1) / op.aux3; }

__device__ __noinline__ void linear_pass(Ctx& c, const OpDesc& op, int tok0, int T, int group, const uint4* pre_w) {
  const KParams& p = c.p;
  const int nkt = op.nkt;
  const int kp = nkt * kTileK;
  const int ntok = min(op.aux3, T - tok0);
  MK_STAMP(c, 0);
  stage_x(c, op.in, op.ld_in, op.k, kp, (op.flags & F_NORM_IN) ? op.norm_w : nullptr, tok0, ntok, T, pre_w,
          MK_XF(op, F_GATHER_IN) != 0);
  MK_STAMP(c, 1);

  const unsigned total = (unsigned)op.nblk * (unsigned)nkt;
  const int G = (int)min(gridDim.x, total);  // with fewer tiles than CTAs the rest idle
  if ((int)blockIdx.x >= G) return;
  const unsigned t0 = tile_begin(blockIdx.x, total, G);
  const unsigned t1 = tile_begin(blockIdx.x + 1, total, G);
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  // A operand: lane l addresses row 16*warp + (l & 7) + 8 * ((l >> 3) & 1), 16-byte chunk 2*kb + (l >> 4)
  const int a_row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t a_base = (uint32_t)(a_row * 128);
  const uint32_t a_xor = (uint32_t)(a_row & 7);
  const uint32_t a_hi = (uint32_t)(lane >> 4);
  // B operand: lane l addresses token (l & 7), chunk 4*half + (l >> 3); absent tokens read the zero chunk
  const int pitch_b = (kp + 8) * 2;
  const bool b_real = (lane & 7) < ntok;
  const uint32_t xs0 = c.smem_addr + p.x_off;
  const uint32_t b_zero = xs0 + (uint32_t)(ntok * pitch_b);
  const uint32_t b_row = xs0 + (uint32_t)((lane & 7) * pitch_b + (lane >> 3) * 16);
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0);

  // The residual element this thread adds first in the epilogue of a row block is requested
  // when the block starts, a whole run of tiles ahead of its use.
  const bool with_res = (op.flags & F_RESIDUAL) && (!(op.flags & F_RES_RANK0) || p.rank == 0);
  const __nv_bfloat16* res_ptr = reinterpret_cast<const __nv_bfloat16*>(op.res) +
                                 (size_t)(tok0 + (c.tid >> 7)) * op.ld_res + (c.tid & 127);
  const bool res_tok = with_res && (c.tid >> 7) < ntok;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int blk = (int)(t0 / (unsigned)nkt);
  int kt = (int)(t0 - (unsigned)blk * (unsigned)nkt);
  int kt_first = kt;
  bool first_of_cta = true;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
  const bool arith = !(p.debug_flags & 1);
  float res0 = 0.f;
  bool new_blk = true;
  for (unsigned tile = t0; tile < t1; ++tile) {
    if (new_blk) {
      new_blk = false;
      res0 = 0.f;
      if (res_tok && blk * kTileRows + (c.tid & 127) < op.n)
        res0 = MK_XF(op, F_GATHER_RES) ? xchg_gather1(c, xchg_cur(c), tok0 + (c.tid >> 7), blk * kTileRows + (c.tid & 127))
                                         : __bfloat162float(__ldcg(res_ptr + blk * kTileRows));
    }
    mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
    if (tile == t0) MK_STAMP(c, 2);
    const uint32_t st = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes + a_base;
    if (arith) {
#pragma unroll
      for (int sub = 0; sub < kSubTiles; ++sub) {
        uint32_t b[8];
        const uint32_t bk = b_real ? b_row + (uint32_t)kt * (kTileK * 2) + (uint32_t)sub * (kBoxK * 2) : b_zero;
        ldmatrix_x4(bk, b[0], b[1], b[2], b[3]);
        ldmatrix_x4(b_real ? bk + 64 : b_zero, b[4], b[5], b[6], b[7]);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(st + (uint32_t)sub * kSubBytes + ((((uint32_t)(2 * kb) + a_hi) ^ a_xor) << 4), a0, a1, a2, a3);
          mma_bf16(acc, a0, a1, a2, a3, b[2 * kb], b[2 * kb + 1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty0 + 8 * s);
    ++consumed;
    if (++s == S) {
      s = 0;
      parity ^= 1u;
    }
    const bool end_blk = (kt == nkt - 1);
    if (tile == t1 - 1) MK_STAMP(c, 3);
    if (end_blk || tile == t1 - 1) {
      // thread (lane) holds rows 16*warp + lane/4 (+8) and tokens 2*(lane%4) (+1)
      float* red = c.sums() + (16 * warp + (lane >> 2)) * p.sums_stride + 2 * (lane & 3);
      red[0] = acc[0];
      red[1] = acc[1];
      red[8 * p.sums_stride] = acc[2];
      red[8 * p.sums_stride + 1] = acc[3];
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      linear_finish_piece(c, op, blk, kt_first, kt, first_of_cta, tok0, ntok, group, res0);
      first_of_cta = false;
      kt_first = 0;
      if (tile == t1 - 1) MK_STAMP(c, 4);
    }
    if (end_blk) {
      kt = 0;
      blk += 1;
      new_blk = true;
    } else {
      kt += 1;
    }
  }
  c.cons_idx += consumed;
}

// Batches above 8 tokens: the input rows of a pass (16, 32 or 64 token rows x 128 k) come
// with every weight stage as two more TMA boxes (issued by the activation producer once the
// op's barrier has opened), 128-byte swizzled like the weights, and each warp multiplies its
// 16 weight rows against NT n-tiles of 8 tokens.  The weights are streamed once per pass of
// up to 64 tokens instead of once per 8.
template <int NT>
__device__ __noinline__ void linear_pass_wide(Ctx& c, const OpDesc& op, int tok0, int T, int group) {
  const KParams& p = c.p;
  const int nkt = op.nkt;
  const int ntok = min(8 * NT, T - tok0);
  const unsigned total = (unsigned)op.nblk * (unsigned)nkt;
  const int G = (int)min(gridDim.x, total);
  if ((int)blockIdx.x >= G) return;
  const unsigned t0 = tile_begin(blockIdx.x, total, G);
  const unsigned t1 = tile_begin(blockIdx.x + 1, total, G);
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  const int a_row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t a_base = (uint32_t)(a_row * 128);
  const uint32_t a_xor = (uint32_t)(a_row & 7);
  const uint32_t a_hi = (uint32_t)(lane >> 4);
  // B operand: lane l addresses token row 8*nt + (l & 7), 16-byte chunk 4*half + (l >> 3)
  const uint32_t b_row = (uint32_t)((lane & 7) * 128);
  const uint32_t b_xor = (uint32_t)(lane & 7);
  const uint32_t b_hi = (uint32_t)(lane >> 3);
  const uint32_t x_sub = (uint32_t)(8 * NT * 128);  // bytes of one activation box
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0), bar_x0 = c.xfull_bar(0);
  const bool with_res = (op.flags & F_RESIDUAL) && (!(op.flags & F_RES_RANK0) || p.rank == 0);
  const __nv_bfloat16* res_ptr = reinterpret_cast<const __nv_bfloat16*>(op.res) +
                                 (size_t)(tok0 + (c.tid >> 7)) * op.ld_res + (c.tid & 127);
  const bool res_tok = with_res && (c.tid >> 7) < ntok;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  int blk = (int)(t0 / (unsigned)nkt);
  int kt = (int)(t0 - (unsigned)blk * (unsigned)nkt);
  int kt_first = kt;
  bool first_of_cta = true;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
  float res0 = 0.f;
  bool new_blk = true;
  for (unsigned tile = t0; tile < t1; ++tile) {
    if (new_blk) {
      new_blk = false;
      res0 = 0.f;
      if (res_tok && blk * kTileRows + (c.tid & 127) < op.n)
        res0 = MK_XF(op, F_GATHER_RES) ? xchg_gather1(c, xchg_cur(c), tok0 + (c.tid >> 7), blk * kTileRows + (c.tid & 127))
                                         : __bfloat162float(__ldcg(res_ptr + blk * kTileRows));
    }
    mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
    mbar_wait(c, bar_x0 + 8 * s, (c.xphase >> s) & 1u, ST_TIMEOUT_FULL);
    c.xphase ^= 1u << s;
    const uint32_t st = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
    const uint32_t xt = st + kStageBytes;
#pragma unroll
    for (int sub = 0; sub < kSubTiles; ++sub) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t a[2][4];
#pragma unroll
        for (int q = 0; q < 2; ++q)
          ldmatrix_x4(st + a_base + (uint32_t)sub * kSubBytes + ((((uint32_t)(2 * (2 * half + q)) + a_hi) ^ a_xor) << 4),
                      a[q][0], a[q][1], a[q][2], a[q][3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(xt + (uint32_t)sub * x_sub + (uint32_t)nt * 1024u + b_row + ((((uint32_t)(4 * half) + b_hi) ^ b_xor) << 4),
                      b0, b1, b2, b3);
          mma_bf16(acc[nt], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
          mma_bf16(acc[nt], a[1][0], a[1][1], a[1][2], a[1][3], b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty0 + 8 * s);
    ++consumed;
    if (++s == S) {
      s = 0;
      parity ^= 1u;
    }
    const bool end_blk = (kt == nkt - 1);
    if (end_blk || tile == t1 - 1) {
      float* red = c.sums() + (16 * warp + (lane >> 2)) * p.sums_stride + 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[8 * nt] = acc[nt][0];
        red[8 * nt + 1] = acc[nt][1];
        red[8 * p.sums_stride + 8 * nt] = acc[nt][2];
        red[8 * p.sums_stride + 8 * nt + 1] = acc[nt][3];
        acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      }
      linear_finish_piece(c, op, blk, kt_first, kt, first_of_cta, tok0, ntok, group, res0);
      first_of_cta = false;
      kt_first = 0;
    }
    if (end_blk) {
      kt = 0;
      blk += 1;
      new_blk = true;
    } else {
      kt += 1;
    }
  }
  c.cons_idx += consumed;
}

// ------------------------------------------------------------------------------------
// Stream-K tiles on the 5th-generation tensor cores (17-64 tokens).  With mma.sync every warp
// re-reads the activation boxes of a stage (at 64 tokens: 160 KB of ldmatrix traffic per
// 32 KB weight tile, the SM's shared-memory bandwidth is the limit).  tcgen05.mma reads both
// operands from shared memory once: A = the weight tile (M = 128 rows), B = the activation
// box (N = 32 or 64 token rows), both K-major with the 128-byte swizzle TMA left them in;
// D = 128 lanes x N columns of fp32 in tensor memory.  One thread issues the 8 MMAs of a
// stage (2 boxes x 4 k-steps of 16) and commits them to the stage's "empty" mbarrier; when a
// run of tiles ends, a commit to the "done" mbarrier tells all warps to fetch the
// accumulators (tcgen05.ld, warp w reads lanes 32 * (w & 3) .. + 31) into the sums block,
// from where the usual split-k finish and epilogue take over.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
  // start address >> 4 | leading offset (unused for swizzled K-major) 1 | stride between 8-row
  // groups 1024 B >> 4 | descriptor version 1 | layout 2 = 128-byte swizzle
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __noinline__ void linear_pass_umma(Ctx& c, const OpDesc& op, int tok0, int T, int group) {
  const KParams& p = c.p;
  const int nkt = op.nkt;
  const int ntok = min(op.aux3, T - tok0);
  const int N = p.x_rows;  // 32 or 64 token rows per activation box
  const unsigned total = (unsigned)op.nblk * (unsigned)nkt;
  const int G = (int)min(gridDim.x, total);
  if ((int)blockIdx.x >= G) return;
  const unsigned t0 = tile_begin(blockIdx.x, total, G);
  const unsigned t1 = tile_begin(blockIdx.x + 1, total, G);
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  const uint32_t x_sub = (uint32_t)N * 128u;  // bytes of one activation box
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0), bar_x0 = c.xfull_bar(0);
  // instruction descriptor: D = f32, A = B = bf16, both K-major, N >> 3, M >> 4
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
  const bool with_res = (op.flags & F_RESIDUAL) && (!(op.flags & F_RES_RANK0) || p.rank == 0);
  const __nv_bfloat16* res_ptr = reinterpret_cast<const __nv_bfloat16*>(op.res) +
                                 (size_t)(tok0 + (c.tid >> 7)) * op.ld_res + (c.tid & 127);
  const bool res_tok = with_res && (c.tid >> 7) < ntok;
  int blk = (int)(t0 / (unsigned)nkt);
  int kt = (int)(t0 - (unsigned)blk * (unsigned)nkt);
  int kt_first = kt;
  bool first_of_cta = true;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
  float res0 = 0.f;
  bool new_blk = true;
  bool fresh = true;  // the next MMA starts a run: it overwrites the accumulators
  for (unsigned tile = t0; tile < t1; ++tile) {
    if (new_blk) {
      new_blk = false;
      res0 = 0.f;
      if (res_tok && blk * kTileRows + (c.tid & 127) < op.n)
        res0 = MK_XF(op, F_GATHER_RES) ? xchg_gather1(c, xchg_cur(c), tok0 + (c.tid >> 7), blk * kTileRows + (c.tid & 127))
                                         : __bfloat162float(__ldcg(res_ptr + blk * kTileRows));
    }
    // every warp follows the ring (one arrival per warp and phase keeps the "empty" count
    // exact); warp 0's arrival is the commit of the stage's MMAs
    bool ok = mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
    if (warp == 0) {
      ok = mbar_wait(c, bar_x0 + 8 * s, (c.xphase >> s) & 1u, ST_TIMEOUT_FULL) && ok;
      if (lane == 0) {
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
          const uint32_t xt = st + kStageBytes;
#pragma unroll
          for (int sub = 0; sub < kSubTiles; ++sub) {
            const uint64_t ad = umma_smem_desc(st + (uint32_t)sub * kSubBytes);
            const uint64_t bd = umma_smem_desc(xt + (uint32_t)sub * x_sub);
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
              // 16 k-elements = 32 bytes further inside the 128-byte swizzle span: +2 in the address field
              umma_bf16(c.tmem, ad + (uint64_t)(2 * k16), bd + (uint64_t)(2 * k16), idesc, (fresh && sub == 0 && k16 == 0) ? 0u : 1u);
            }
          }
          umma_commit(bar_empty0 + 8 * s);
        } else {
          mbar_arrive(bar_empty0 + 8 * s);  // aborting: keep the count exact, the body is skipped
        }
      }
      __syncwarp();
    } else if (lane == 0) {
      mbar_arrive(bar_empty0 + 8 * s);
    }
    c.xphase ^= 1u << s;
    fresh = false;
    ++consumed;
    if (++s == S) {
      s = 0;
      parity ^= 1u;
    }
    const bool end_blk = (kt == nkt - 1);
    if (end_blk || tile == t1 - 1) {
      // accumulators complete -> sums block [row][token]
      if (warp == 0 && lane == 0) umma_commit(c.done_bar());
      __syncwarp();
      mbar_wait(c, c.done_bar(), c.done_phase & 1u, ST_TIMEOUT_FULL);
      c.done_phase += 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __syncwarp();
      {
        const int q = warp & 3, half = warp >> 2;  // lane quadrant, column half
        const int row = 32 * q + lane;
        const int ncol = N >> 1;  // columns of this warp: 16 or 32
        float* dst = c.sums() + row * p.sums_stride + half * ncol;
#pragma unroll 1
        for (int c0 = 0; c0 < ncol; c0 += 16) {
          float v[16];
          tmem_ld16(c.tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(half * ncol + c0), v);
#pragma unroll
          for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(dst + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      linear_finish_piece(c, op, blk, kt_first, kt, first_of_cta, tok0, ntok, group, res0);
      first_of_cta = false;
      kt_first = 0;
      fresh = true;
    }
    if (end_blk) {
      kt = 0;
      blk += 1;
      new_blk = true;
    } else {
      kt += 1;
    }
  }
  c.cons_idx += consumed;
}

// ------------------------------------------------------------------------------------
// Row-owner linear (F_ROWS): for one or two tokens the cross-CTA finish of a k-split costs
// more than the whole weight stream of a small layer, so every CTA takes whole output rows
// instead: a contiguous range of 8-row units, walked in chunks of up to 32 rows over the
// full K.  The token rows are resident in shared memory (stage_x, fused norm included).
// Inside a chunk the 8 warps split k: warp w multiplies the w-th 64-wide k slice of every
// 512-wide stage, 16 weight rows on the M side of the mma and the tokens on the N side, and
// the eight partial sums of an output meet in shared memory when the chunk ends.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void rows_range(const OpDesc& op, int& row0, int& row1, bool& any) {
  const unsigned U = (unsigned)(op.n + kUnitRows - 1) / kUnitRows;
  const unsigned G = min((unsigned)gridDim.x, U);
  any = blockIdx.x < G;
  row0 = any ? (int)tile_begin(blockIdx.x, U, G) * kUnitRows : 0;
  row1 = any ? (int)tile_begin(blockIdx.x + 1, U, G) * kUnitRows : 0;
}
// The CTA's rows are walked in chunks of at most 32 rows, sized as evenly as whole 8-row units
// allow (40 rows are 24 + 16, not 32 + 8: small chunks mean small stages and few bytes in
// flight).  Chunk ci of nch covers rows [rows_chunk_begin(ci), rows_chunk_begin(ci + 1)).
__device__ __forceinline__ int rows_num_chunks(int row0, int row1) { return (row1 - row0 + kChunkRows - 1) / kChunkRows; }
__device__ __forceinline__ int rows_chunk_begin(int row0, int row1, int nch, int ci) {
  return row0 + kUnitRows * (ci * ((row1 - row0) / kUnitRows) / nch);
}
// weight stages of this CTA in one pass of the op
__device__ __forceinline__ unsigned rows_stage_count(const OpDesc& op) {
  int row0, row1;
  bool any;
  rows_range(op, row0, row1, any);
  return (unsigned)((row1 - row0 + kChunkRows - 1) / kChunkRows) * (unsigned)op.nkt;
}

__device__ __noinline__ void linear_pass_rows(Ctx& c, const OpDesc& op, int tok0, int T, const uint4* pre_w) {
  const KParams& p = c.p;
  const int nks = op.nkt;
  const int kp = nks * kRowsStageK;
  const int ntok = min(op.aux3, T - tok0);
  MK_STAMP(c, 0);
  if (op.flags & F_LL_IN) {
    if (op.flags & F_NORM_IN) stage_x_ll(c, op.ll_in, op.ld_in, op.k, kp, op.norm_w, tok0, ntok, T, pre_w, ll_tag_of(c, op.ll_in_op));
    else stage_rows_ll(c, op.ll_in, op.ld_in, op.k, kp, tok0, ntok, T, ll_tag_of(c, op.ll_in_op));
  } else if (nks <= 24 && ntok <= 2 && !(op.flags & F_NORM_IN) && !MK_XF(op, F_GATHER_IN)) stage_x_rows(c, op.in, op.ld_in, op.k, kp, tok0, ntok, T);
  else stage_x(c, op.in, op.ld_in, op.k, kp, (op.flags & F_NORM_IN) ? op.norm_w : nullptr, tok0, ntok, T, pre_w,
               MK_XF(op, F_GATHER_IN) != 0);
  MK_STAMP(c, 1);
  int row0, row1;
  bool any;
  rows_range(op, row0, row1, any);
  if (!any) return;
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  const bool arith = !(p.debug_flags & 1);
  // B operand (k x tokens): lane l addresses token (l & 7), 16-byte chunk (l >> 3) of a 32-wide k step
  const int pitch_b = (kp + 8) * 2;
  const uint32_t xs0 = c.smem_addr + p.x_off;
  const bool a_real = (lane & 7) < ntok;
  const uint32_t a_row = a_real ? xs0 + (uint32_t)((lane & 7) * pitch_b + (lane >> 3) * 16 + warp * 128)
                                : xs0 + (uint32_t)(ntok * pitch_b);  // the zero chunk
  // Weights sit on the M side of the mma (16 rows per tile, so a 32-row chunk is two tiles of
  // four k steps: half the instructions of 8-row tiles on the N side) and the tokens on the N
  // side.  Lane l addresses row (l & 15) of a tile and the 16-byte chunk 2 * step + (l >> 4)
  // of the warp's 128-byte-swizzled box.
  const uint32_t w_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
  const uint32_t w_xor = (uint32_t)(lane & 7);
  const uint32_t w_hi = (uint32_t)(lane >> 4);
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0);
  const int TP = p.sums_stride;  // token slots of the sums block: [warp][32 rows][TP]
  float* sums = c.sums();
  const bool with_res = (op.flags & F_RESIDUAL) && (!(op.flags & F_RES_RANK0) || p.rank == 0);
  const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(op.res);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  // epilogue role of this thread: output (row e & 31, token e >> 5) of the chunk
  const int e_row = c.tid & 31, e_tok = c.tid >> 5;
  ArgBest best;  // F_ARGMAX: lane 0 of warp t keeps the running best of token t over the CTA's rows
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
  const int nch = rows_num_chunks(row0, row1);
#pragma unroll 1
  for (int ci = 0; ci < nch; ++ci) {
    const int r0 = rows_chunk_begin(row0, row1, nch, ci);
    const int R = rows_chunk_begin(row0, row1, nch, ci + 1) - r0;
    const int ntile = (R + 15) >> 4;  // a ragged last tile reads 8 rows of bytes behind the box: ignored rows
    // the residual of this thread's output is requested a whole chunk ahead of its use
    float res0 = 0.f;
    const bool e_live = e_row < R && e_tok < ntok && r0 + e_row < op.n;
    if (with_res && e_live) {
      if (op.flags & F_LL_RES) res0 = ll_gather1(c, ll_row(op.ll_res, op.ld_res, tok0 + e_tok), r0 + e_row, ll_tag_of(c, op.ll_res_op));
      else res0 = MK_XF(op, F_GATHER_RES) ? xchg_gather1(c, xchg_cur(c), tok0 + e_tok, r0 + e_row)
                                            : __bfloat162float(__ldcg(res + (size_t)(tok0 + e_tok) * op.ld_res + r0 + e_row));
    }
    float acc[4][4];  // [2 * tile + (k step & 1)]: two chains per tile, added up at the end
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    const uint32_t box_bytes = (uint32_t)R * 128u;
#pragma unroll 1
    for (int ks = 0; ks < nks; ++ks) {
      if (ks == 0 && ci == 0) MK_STAMP(c, 2);
      mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
      if (arith) {
        const uint32_t wb = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes + (uint32_t)warp * box_bytes + w_off;
        const uint32_t xa = a_row + (a_real ? (uint32_t)(ks * kRowsStageK * 2) : 0u);
        uint32_t x[2][4];  // x[h]: k chunks 4h .. 4h+3 of tokens 0..7: the B fragments of k steps 2h and 2h+1
        ldmatrix_x4(xa, x[0][0], x[0][1], x[0][2], x[0][3]);
        ldmatrix_x4(xa + (a_real ? 64u : 0u), x[1][0], x[1][1], x[1][2], x[1][3]);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (t < ntile) {
#pragma unroll
            for (int st = 0; st < 4; ++st) {
              uint32_t w0, w1, w2, w3;
              ldmatrix_x4(wb + (uint32_t)t * 2048u + ((((uint32_t)(2 * st) + w_hi) ^ w_xor) << 4), w0, w1, w2, w3);
              mma_bf16(acc[2 * t + (st & 1)], w0, w1, w2, w3, x[st >> 1][2 * (st & 1)], x[st >> 1][2 * (st & 1) + 1]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty0 + 8 * s);
      ++consumed;
      if (++s == S) {
        s = 0;
        parity ^= 1u;
      }
    }
    if (ci == nch - 1) MK_STAMP(c, 3);
    // the chunk's partial sums of this warp: rows 16t + (lane >> 2) and + 8, tokens 2 * (lane & 3) + {0, 1}
    {
      const int tk = 2 * (lane & 3);
      if (tk < TP) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          float* d = sums + ((warp * kChunkRows + 16 * t + (lane >> 2)) * TP + tk);
          d[0] = acc[2 * t][0] + acc[2 * t + 1][0];
          d[8 * TP] = acc[2 * t][2] + acc[2 * t + 1][2];
          if (tk + 1 < TP) {
            d[1] = acc[2 * t][1] + acc[2 * t + 1][1];
            d[8 * TP + 1] = acc[2 * t][3] + acc[2 * t + 1][3];
          }
        }
      }
    }
    consumer_sync();
    if (op.flags & F_SILU_MUL) {
      // units are [4 gate rows | 4 up rows]: the thread of a gate row also adds up its partner
      const int col = ((r0 + e_row) >> 3) * 4 + (e_row & 3);
      const bool mine = (e_row & 7) < 4 && e_live && col < (op.n >> 1);
      __nv_bfloat16 y = __float2bfloat16_rn(0.f);
      if (mine) {
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int w = 0; w < kNumConsumerWarps; ++w) {
          g += sums[(w * kChunkRows + e_row) * TP + e_tok];
          u += sums[(w * kChunkRows + e_row + 4) * TP + e_tok];
        }
        g = rbf(g);  // the linear output is bf16 before the activation
        u = rbf(u);
        const float sv = rbf(__fdividef(g, 1.0f + __expf(-g)));
        y = __float2bfloat16_rn(sv * u);
        out[(size_t)(tok0 + e_tok) * op.ld_out + col] = y;
      }
      if (op.flags & F_LL_OUT) {  // the pair (col, col + 1) sits in two neighbouring lanes
        const uint32_t lo = (uint32_t)__bfloat16_as_ushort(y);
        const uint32_t hi = __shfl_down_sync(0xffffffffu, lo, 1);
        if (mine && !(e_row & 1))
          st_gpu_v2(reinterpret_cast<uint2*>(op.ll_out) + (size_t)(tok0 + e_tok) * (size_t)(op.ld_out >> 1) + (col >> 1), lo | (hi << 16),
                    ll_tag_of(c, c.cur_op));
      }
    } else {
      float v = 0.f;
      if (e_live) {
#pragma unroll
        for (int w = 0; w < kNumConsumerWarps; ++w) v += sums[(w * kChunkRows + e_row) * TP + e_tok];
        if (with_res) v = (p.numerics == NUM_TORCH && !MK_XF(op, F_PUSH)) ? rbf(v) + res0 : v + res0;
        if (MK_XF(op, F_PUSH)) xchg_push1(p, xchg_next(c), tok0 + e_tok, r0 + e_row, v);
        else out[(size_t)(tok0 + e_tok) * op.ld_out + r0 + e_row] = __float2bfloat16_rn(v);
      }
      if (op.flags & F_LL_OUT) {  // rows come in units of 8: the pair (row, row + 1) sits in two neighbouring lanes
        const uint32_t lo = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
        const uint32_t hi = __shfl_down_sync(0xffffffffu, lo, 1);
        if (e_live && !(e_row & 1))
          st_gpu_v2(reinterpret_cast<uint2*>(op.ll_out) + (size_t)(tok0 + e_tok) * (size_t)(op.ld_out >> 1) + ((r0 + e_row) >> 1),
                    lo | (hi << 16), ll_tag_of(c, c.cur_op));
      }
      if (op.flags & F_ARGMAX) {
        ArgBest b;
        b.v = e_live ? rbf(v) : -INFINITY;
        b.i = e_live ? r0 + e_row : 0x7fffffff;
        b = warp_argmax(b);
        best = arg_better(best, b);
      }
    }
    if (ci + 1 < nch) consumer_sync();  // the sums block is free again (after the last chunk, the sync that opens the next op or pass does it)
  }
  if ((op.flags & F_ARGMAX) && lane == 0 && e_tok < ntok) {
    op.amax_val[(size_t)(tok0 + e_tok) * op.amax_n + blockIdx.x] = best.v;
    op.amax_idx[(size_t)(tok0 + e_tok) * op.amax_n + blockIdx.x] = best.i;
  }
  MK_STAMP(c, 4);
  c.cons_idx += consumed;
}

template <int PATH>
__device__ void op_linear(Ctx& c, const OpDesc& op, int T) {
  // the norm weights do not depend on other CTAs: fetched ahead of the barrier
  uint4 pre_w[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  bool pre = false;
  if constexpr (PATH != PATH_UMMA) {
    const int wpr0 = stage_warps_per_row(min(op.aux3, T));
    const int kvec_pad = op.nkt * ((PATH == PATH_ROWS ? kRowsStageK : kTileK) >> 3);  // padded row, in 16-byte vectors
    pre = (op.flags & F_NORM_IN) && kvec_pad <= 128 * wpr0;
    if (pre) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = (c.warp % wpr0) * 32 + c.lane + 32 * wpr0 * i;
        if (v < (op.k >> 3)) pre_w[i] = __ldg(reinterpret_cast<const uint4*>(op.norm_w) + v);
      }
    }
  }
#if MK_WITH_XCHG
  if (op.flags & F_XRED) xchg_reduce_slice(c, op, T);
#endif
  if (op.flags & F_LL_IN) {
    // No barrier, and no look at the abort flag either (a round trip to L2 per op): the polls of the
    // tagged input and the stage waits watch it, and an aborted iteration ends at its closing barrier.
    if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
  } else if (op_barrier(c, op)) {
    return;
  }
  c.lin_seq += 1;
  if (c.tid == 0) c.flags()[4] = (int)c.lin_seq;  // the activation producer may now read this op's input
  const int passes = linear_passes(op, T);
  if constexpr (PATH == PATH_ROWS) {
    for (int g = 0; g < passes; ++g) {
      linear_pass_rows(c, op, g * op.aux3, T, (pre && g == 0) ? pre_w : nullptr);
      if (g + 1 < passes) consumer_sync();  // (a pass leaves its last chunk's sums block without a sync of its own)
    }
  } else if constexpr (PATH == PATH_UMMA) {
    for (int g = 0; g < passes; ++g) linear_pass_umma(c, op, g * op.aux3, T, g);
  } else {
    if (op.flags & F_XTILE) {
      for (int g = 0; g < passes; ++g) {
        if (c.p.x_rows == 8) linear_pass_wide<1>(c, op, g * op.aux3, T, g);
        else linear_pass_wide<2>(c, op, g * op.aux3, T, g);
      }
    } else {
      for (int g = 0; g < passes; ++g) linear_pass(c, op, g * op.aux3, T, g, (pre && g == 0) ? pre_w : nullptr);
    }
  }
  if (MK_XF(op, F_PUSH)) c.ar_seq += 1;  // every CTA counts the exchange, with or without rows of its own
}

// ------------------------------------------------------------------------------------
// attention: QK-norm + RoPE + KV append + paged split-KV GQA decode + merge
// ------------------------------------------------------------------------------------
// Work split inside a CTA: warp w serves q head (w % qpk) of the task's kv-head group and
// position group (w / qpk); its two half-warps take alternate positions.  One head
// vector is spread over the 16 lanes of a half-warp, 8 dims each, so a cached K or V
// row of 256 bytes is one 16-byte load per lane.  The code is kept small on purpose:
// the megakernel switches between task bodies thousands of times per step and every
// switch refills the instruction cache.

// bf16 reciprocal square root the way the reference PyTorch model's CPU kernels round it:
// `dbl` = scalar loop (sqrt rounded to bf16 before the reciprocal), else vector loop.
__device__ __noinline__ float torch_rsqrt_bf16(float var, bool dbl) {
  return dbl ? rbf(1.0f / rbf(sqrtf(var))) : rbf(1.0f / sqrtf(var));
}

// The norm weight and the cos/sin rows arrive already loaded (8 bf16 each).  Both halves
// of a warp run this with full-mask shuffles (xor < 16 stays inside a half-warp).
struct F8 {
  float v[8];
};
__device__ __noinline__ F8 head_norm_rope(F8 xin, uint4 wv, uint4 csv, uint4 snv, int l16, int flags, int numerics,
                                          bool dbl) {
  float* x = xin.v;
  if (flags & F_QK_NORM) {
    float w[8];
    unpack8(wv, w);
    float ss = 0.f;
    if (numerics == NUM_TORCH) {
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += rbf(x[i] * x[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (numerics == NUM_TORCH) {
      const float r = torch_rsqrt_bf16(rbf(ss / (float)kHeadDim), dbl);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = rbf(w[i] * rbf(x[i] * r));
    } else {
      const float r = rsqrtf(ss / (float)kHeadDim + 1e-6f);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = rbf(x[i] * (r * w[i]));
    }
  }
  if (flags & F_ROPE) {
    float cs[8], sn[8];
    unpack8(csv, cs);
    unpack8(snv, sn);
    const float sign = (l16 < 8) ? -1.f : 1.f;  // first half: x*cos - partner*sin
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 8);
      if (numerics == NUM_TORCH) x[i] = rbf(rbf(x[i] * cs[i]) + rbf(sign * other * sn[i]));
      else x[i] = rbf(x[i] * cs[i] + sign * other * sn[i]);
    }
  }
  return xin;
}

// Everything a (token, kv head, chunk) task needs that does not depend on the QKV
// rows of this layer: lengths, page numbers, norm weights, cos/sin, and the first
// four cached K/V rows of this half-warp.  Loaded before the op's grid barrier for
// the CTA's first task, so that only the q path is left on the critical path.
struct AttnTask {
  int t, h, ch, L, p0, p1, nch, kv_base, new_page;
  bool valid;
  uint4 wq, wk, cs, sn;
  uint4 kr[4], vr[4];
};

constexpr int kAttnLensMax = 128;  // requests (the host admits at most 128 batched tokens)

struct AttnPlan {
  int HKV, qpk, CS, nch_max, ntasks;
  int gi, ngroups;  // this half-warp's position group and the number of groups
};

// rows of positions p0 + (it0 + u) * ngroups + gi, u = 0..3
// `pgc`: this half-warp's four cached page numbers (the metadata of an iteration is the same
// for all layers, so only the first attention op of an iteration looks them up: `fill`).
// `pgs`: when not null, the page numbers of page slots (a.p0 >> page_shift) + 0..15 of the request,
// cached in shared memory (the row loop would otherwise wait for a page look-up before every load).
__device__ __forceinline__ void attn_fetch_rows(const Ctx& c, const OpDesc& op, const AttnPlan& pl, const AttnTask& a,
                                                int it0, int l16, uint4* kr, uint4* vr, int* pgc = nullptr,
                                                bool fill = false, const int* pgs = nullptr) {
  const int psh = c.p.page_shift, pmask = c.p.page_size - 1;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int j = a.p0 + (it0 + u) * pl.ngroups + pl.gi;
    kr[u] = make_uint4(0, 0, 0, 0);
    vr[u] = make_uint4(0, 0, 0, 0);
    if (j < a.p1 && j != a.L - 1) {
      int pg;
      const int slot = (j >> psh) - (a.p0 >> psh);
      if (pgc != nullptr && !fill) {
        pg = pgc[u];
      } else if (pgs != nullptr && slot < 16) {
        pg = pgs[slot];
      } else {
        pg = __ldcg(c.p.kv_indices + a.kv_base + (j >> psh));
        if (pgc != nullptr) pgc[u] = pg;  // all 16 lanes store the same number
      }
      const size_t src = ((((size_t)pg << psh) + (j & pmask)) * pl.HKV + a.h) * kHeadDim;
      kr[u] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.k_cache) + src) + l16);
      vr[u] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.v_cache) + src) + l16);
    }
  }
}

// NORMW: also fetch the norm weights and the cos/sin row of the task's position (the single-task path fetches
// them itself, next to the q/k rows: held from here on, they were spilled, and a spill waits for its load).
template <bool NORMW = true, bool FETCH = true>
__device__ __forceinline__ void attn_prepare(const Ctx& c, const OpDesc& op, const AttnPlan& pl, const int* lens, int task,
                                          int l16, AttnTask& a, int* pgc = nullptr, bool fill = false,
                                          int* geom = nullptr) {
  // `geom`: the task's geometry as the iteration's first attention op worked it out
  // ([0] valid, then t, h, ch, L, p0, p1, nch, kv_base): the other layers skip the divisions.
  if (geom != nullptr && !fill) {
    a.valid = geom[0] != 0;
    if (!a.valid) return;
    a.t = geom[1]; a.h = geom[2]; a.ch = geom[3]; a.L = geom[4];
    a.p0 = geom[5]; a.p1 = geom[6]; a.nch = geom[7]; a.kv_base = geom[8];
  } else {
    a.valid = false;
    if (geom != nullptr && c.tid == 0) geom[0] = 0;
    if (task >= pl.ntasks) return;
    a.ch = task % pl.nch_max;
    a.h = (task / pl.nch_max) % pl.HKV;
    a.t = task / (pl.nch_max * pl.HKV);
    a.L = lens[a.t];
    a.p0 = a.ch * pl.CS;
    if (a.p0 >= a.L || a.L <= 0) return;
    a.valid = true;
    a.p1 = min(a.L, a.p0 + pl.CS);
    a.nch = (a.L + pl.CS - 1) / pl.CS;
    a.kv_base = lens[kAttnLensMax + a.t];
    if (geom != nullptr && c.tid == 0) {
      geom[0] = 1;
      geom[1] = a.t; geom[2] = a.h; geom[3] = a.ch; geom[4] = a.L;
      geom[5] = a.p0; geom[6] = a.p1; geom[7] = a.nch; geom[8] = a.kv_base;
    }
  }
  if constexpr (NORMW) {
    const int pos = min(a.L - 1, op.aux2 - 1);  // aux2 = rows of the cos/sin tables
    a.wq = __ldg(reinterpret_cast<const uint4*>(op.q_norm_w) + l16);
    a.wk = __ldg(reinterpret_cast<const uint4*>(op.k_norm_w) + l16);
    a.cs = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.cos) + (size_t)pos * kHeadDim) + l16);
    a.sn = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.sin) + (size_t)pos * kHeadDim) + l16);
  }
  if (pgc != nullptr && !fill) {
    a.new_page = pgc[4];
  } else {
    a.new_page = (a.p1 == a.L) ? __ldcg(c.p.kv_indices + a.kv_base + ((a.L - 1) >> c.p.page_shift)) : 0;
    if (pgc != nullptr) pgc[4] = a.new_page;
  }
  if constexpr (FETCH) attn_fetch_rows(c, op, pl, a, 0, l16, a.kr, a.vr, pgc, fill);
}

// Merge of a (request, kv head)'s chunks by the CTA that arrived last: kept out of line, only a
// handful of CTAs per layer ever run it.  One round of loads: every thread fetches, for its
// output elements, the chunks' values together with their (max, sum) pairs and rescales as it
// goes, eight chunks at a time (more loads in flight per thread measured slower).
__device__ __noinline__ void attn_merge(Ctx& c, const float* base, __nv_bfloat16* out, int nch, int qpk, int part_stride,
                                        uint2* ll_out, unsigned tag) {
  const int nout = qpk * kHeadDim;
  constexpr int kMergeBatch = 8;
  // a thread merges outputs e and e + 256 side by side: one round of loads for up to eight chunks of both
#pragma unroll 1
  for (int e = c.tid; e < nout; e += 2 * kNumConsumers) {
    const bool two = e + kNumConsumers < nout;
    const int e2 = two ? e + kNumConsumers : e;
    const float* pm = base + nout + (e >> 7);
    const float* pm2 = base + nout + (e2 >> 7);
    float M = -INFINITY, Ls = 0.f, O = 0.f, M2 = -INFINITY, Ls2 = 0.f, O2 = 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < nch; c0 += kMergeBatch) {
      float v[kMergeBatch], mm[kMergeBatch], ll[kMergeBatch], v2[kMergeBatch], mm2[kMergeBatch], ll2[kMergeBatch];
#pragma unroll
      for (int u = 0; u < kMergeBatch; ++u) {
        const bool ok = c0 + u < nch;
        const size_t off = (size_t)(c0 + u) * part_stride;
        v[u] = ok ? __ldcg(base + off + e) : 0.f;
        mm[u] = ok ? __ldcg(pm + off) : -INFINITY;
        ll[u] = ok ? __ldcg(pm + off + qpk) : 0.f;
        v2[u] = ok ? __ldcg(base + off + e2) : 0.f;
        mm2[u] = ok ? __ldcg(pm2 + off) : -INFINITY;
        ll2[u] = ok ? __ldcg(pm2 + off + qpk) : 0.f;
      }
      float Mb = M, Mb2 = M2;
#pragma unroll
      for (int u = 0; u < kMergeBatch; ++u) {
        Mb = fmaxf(Mb, mm[u]);
        Mb2 = fmaxf(Mb2, mm2[u]);
      }
      const float r = exp2f(M - Mb), r2 = exp2f(M2 - Mb2);  // 0 for the first batch (every chunk holds at least one position)
      O *= r;
      Ls *= r;
      O2 *= r2;
      Ls2 *= r2;
#pragma unroll
      for (int u = 0; u < kMergeBatch; ++u) {
        const float f = exp2f(mm[u] - Mb), f2 = exp2f(mm2[u] - Mb2);
        O = fmaf(f, v[u], O);
        Ls = fmaf(f, ll[u], Ls);
        O2 = fmaf(f2, v2[u], O2);
        Ls2 = fmaf(f2, ll2[u], Ls2);
      }
      M = Mb;
      M2 = Mb2;
    }
    const __nv_bfloat16 y = __float2bfloat16_rn(__fdividef(O, Ls)), y2 = __float2bfloat16_rn(__fdividef(O2, Ls2));
    out[e] = y;
    if (two) out[e2] = y2;
    if (ll_out != nullptr) {  // (whole warps take the same trips: nout is a multiple of 128)
      const uint32_t lo = (uint32_t)__bfloat16_as_ushort(y), lo2 = (uint32_t)__bfloat16_as_ushort(y2);
      const uint32_t hi = __shfl_down_sync(0xffffffffu, lo, 1), hi2 = __shfl_down_sync(0xffffffffu, lo2, 1);
      if (!(e & 1)) {
        st_gpu_v2(ll_out + (e >> 1), lo | (hi << 16), tag);
        if (two) st_gpu_v2(ll_out + (e2 >> 1), lo2 | (hi2 << 16), tag);
      }
    }
  }
}

// The merge without a counter: every chunk stores its partial (output sums, then max and sum per q head) as
// tagged 8-byte words, and every chunk CTA then merges its own slice of the output elements, polling the
// words of all chunks it needs: no atomic round trip, no last arriver doing all of it, one output per
// thread.  (A CTA stores its own partial before it waits for any other, and the chunks of one pair are
// consecutive tasks, so a wait never depends on a later task of the waiting CTA.)
__device__ __noinline__ float ll_wait_word(const Ctx& c, const uint2* w, unsigned tag) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    const uint2 q = ld_gpu_v2(w);
    if (q.y == tag) return __uint_as_float(q.x);
    if (((++spins) & 63u) == 0) {
      if (aborted(c)) return 0.f;
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 2 * c.p.timeout_ns) {
        raise_abort(c, ST_TIMEOUT_DATA, (int)tag, (int)q.y);
        return 0.f;
      }
    }
  }
}
__device__ __noinline__ void attn_merge_ll(Ctx& c, const uint2* base, __nv_bfloat16* out, uint2* ll_out, int nch, int ch, int qpk,
                                           int part_stride, unsigned tag) {
  const int nout = qpk * kHeadDim;
  const int S = (((nout + nch - 1) / nch) + 1) & ~1;  // outputs per chunk CTA, even: a bf16 pair never straddles two slices
#pragma unroll 1
  for (int el0 = 0; el0 < S; el0 += kNumConsumers) {  // (one round for up to four q heads per kv head)
    const int el = el0 + c.tid;
    const int e = ch * S + el;
    const bool act = el < S && e < nout;
    float y = 0.f;
    if (act) {
      constexpr int kBatch = 8;
      const uint2* pv = base + e;
      const uint2* pm = base + nout + (e >> 7);
      float M = -INFINITY, Ls = 0.f, O = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < nch; c0 += kBatch) {
        uint2 qv[kBatch], qm[kBatch], ql[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const bool ok = c0 + u < nch;
          const size_t off = (size_t)(ok ? c0 + u : c0) * part_stride;
          qv[u] = ld_gpu_v2(pv + off);
          qm[u] = ld_gpu_v2(pm + off);
          ql[u] = ld_gpu_v2(pm + off + qpk);
        }
        float v[kBatch], mm[kBatch], ll[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const bool ok = c0 + u < nch;
          const size_t off = (size_t)(ok ? c0 + u : c0) * part_stride;
          v[u] = qv[u].y == tag ? __uint_as_float(qv[u].x) : ll_wait_word(c, pv + off, tag);
          mm[u] = qm[u].y == tag ? __uint_as_float(qm[u].x) : ll_wait_word(c, pm + off, tag);
          ll[u] = ql[u].y == tag ? __uint_as_float(ql[u].x) : ll_wait_word(c, pm + off + qpk, tag);
          if (!ok) {
            v[u] = 0.f;
            mm[u] = -INFINITY;
            ll[u] = 0.f;
          }
        }
        float Mb = M;
#pragma unroll
        for (int u = 0; u < kBatch; ++u) Mb = fmaxf(Mb, mm[u]);
        const float r = exp2f(M - Mb);  // 0 for the first batch (every chunk holds at least one position)
        O *= r;
        Ls *= r;
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const float f = exp2f(mm[u] - Mb);
          O = fmaf(f, v[u], O);
          Ls = fmaf(f, ll[u], Ls);
        }
        M = Mb;
      }
      y = __fdividef(O, Ls);
    }
    const __nv_bfloat16 yb = __float2bfloat16_rn(y);
    if (act) out[e] = yb;
    const uint32_t lo = (uint32_t)__bfloat16_as_ushort(yb);
    const uint32_t hi = __shfl_down_sync(0xffffffffu, lo, 1);
    if (act && ll_out != nullptr && !(e & 1)) st_gpu_v2(ll_out + (e >> 1), lo | (hi << 16), tag);
  }
}

// The half-warp's pass over its positions of the task: for up to four q heads of the kv-head
// group, running (max, sum, output) per head.  Rows are consumed four at a time while the next
// four are in flight; `a.kr/a.vr` hold the first batch (loaded ahead of the op's barrier).
__device__ __forceinline__ void attn_rows(const Ctx& c, const OpDesc& op, const AttnPlan& pl, AttnTask& a, int l16, int hq,
                                          const uint4* qv, uint4 knew, uint4 vnew, float sc, float* m, float* l,
                                          float (*o)[8]) {
  const int L = a.L;
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[h][i] = 0.f;
  }
  const int niter = (a.p1 - a.p0 + pl.ngroups - 1) / pl.ngroups;
#pragma unroll 1
  for (int it = 0; it < niter; it += 4) {
    // the next four rows are requested before this batch is used
    uint4 nk[4], nv[4];
    const bool more = it + 4 < niter;
    if (more) attn_fetch_rows(c, op, pl, a, it + 4, l16, nk, nv);
    // The row loop stays rolled (this code runs once per layer out of a cold instruction
    // cache; its size is its cost): the batch's rows are rotated through slot 0 instead of
    // being indexed.
#pragma unroll 1
    for (int u = 0; u < 4; ++u) {
      const int j = a.p0 + (it + u) * pl.ngroups + pl.gi;
      const bool ok = j < a.p1;  // may differ between the two halves of a warp: no shuffle may depend on it
      if (__any_sync(0xffffffffu, ok)) {
        uint4 kr = a.kr[0], vr = a.vr[0];
        if (ok && j == L - 1) {
          kr = knew;
          vr = vnew;
        }
        float kk[8], vf[8];
        unpack8(kr, kk);
        unpack8(vr, vf);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          if (h < hq) {  // uniform
            float qf[8];
            unpack8(qv[h], qf);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) d = fmaf(qf[i], kk[i], d);
#pragma unroll
            for (int x = 8; x > 0; x >>= 1) d += __shfl_xor_sync(0xffffffffu, d, x);
            if (ok) {
              const float sv = d * sc;
              const float mn = fmaxf(m[h], sv);
              const float alpha = exp2f(m[h] - mn), pr = exp2f(sv - mn);
              l[h] = l[h] * alpha + pr;
#pragma unroll
              for (int i = 0; i < 8; ++i) o[h][i] = fmaf(pr, vf[i], o[h][i] * alpha);
              m[h] = mn;
            }
          }
        }
      }
      a.kr[0] = a.kr[1]; a.kr[1] = a.kr[2]; a.kr[2] = a.kr[3];
      a.vr[0] = a.vr[1]; a.vr[1] = a.vr[2]; a.vr[2] = a.vr[3];
    }
    if (more) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a.kr[u] = nk[u];
        a.vr[u] = nv[u];
      }
    }
  }
}

// The same pass for ONE q head per half-warp (the single-chunk-per-CTA path): running
// (max, sum, output) of the half-warp's positions of the task.  Four rows are handled as one
// batch: their dot products and the four shuffle trees run side by side, and the running
// maximum is updated once per batch, so the dependent chain of a batch is about as long as
// that of a single row.  `pgs`: see attn_fetch_rows.
__device__ __forceinline__ void attn_rows1(const Ctx& c, const OpDesc& op, const AttnPlan& pl, AttnTask& a, int l16,
                                           uint4 qv, uint4 knew, uint4 vnew, float sc, float& m, float& l, float* o,
                                           const int* pgs) {
  const int L = a.L;
  m = -INFINITY;
  l = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = 0.f;
  float qf[8];
  unpack8(qv, qf);
  const int niter = (a.p1 - a.p0 + pl.ngroups - 1) / pl.ngroups;
#pragma unroll 1
  for (int it = 0; it < niter; it += 4) {
    uint4 nk[4], nv[4];  // the next four rows are requested before this batch is used
    const bool more = it + 4 < niter;
    if (more) attn_fetch_rows(c, op, pl, a, it + 4, l16, nk, nv, nullptr, false, pgs);
    float sv[4];
    bool ok[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = a.p0 + (it + u) * pl.ngroups + pl.gi;
      ok[u] = j < a.p1;  // may differ between the two halves of a warp: the shuffles below do not depend on it
      if (ok[u] && j == L - 1) {
        a.kr[u] = knew;
        a.vr[u] = vnew;
      }
      float kk[8];
      unpack8(a.kr[u], kk);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) d = fmaf(qf[i], kk[i], d);
      sv[u] = d;
    }
#pragma unroll
    for (int x = 8; x > 0; x >>= 1) {
#pragma unroll
      for (int u = 0; u < 4; ++u) sv[u] += __shfl_xor_sync(0xffffffffu, sv[u], x);
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      sv[u] = ok[u] ? sv[u] * sc : -INFINITY;
      mn = fmaxf(mn, sv[u]);
    }
    if (mn != -INFINITY) {  // (a batch without a position of this half-warp leaves everything as it is)
      const float alpha = exp2f(m - mn);
      float pr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) pr[u] = exp2f(sv[u] - mn);
      l = l * alpha + ((pr[0] + pr[1]) + (pr[2] + pr[3]));
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= alpha;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float vf[8];
        unpack8(a.vr[u], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf(pr[u], vf[i], o[i]);
      }
      m = mn;
    }
    if (more) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a.kr[u] = nk[u];
        a.vr[u] = nv[u];
      }
    }
  }
}

// Rows of the task beyond the first four per half-warp (those are loaded into registers) are
// requested into L2 ahead of the op's barrier, one row per lane, so that the row loop's own
// loads find them there.
__device__ __forceinline__ void attn_l2_ahead(const Ctx& c, const OpDesc& op, const AttnPlan& pl, const AttnTask& a, int l16,
                                              const int* pgs) {
  const int psh = c.p.page_shift, pmask = c.p.page_size - 1;
  const int niter = (a.p1 - a.p0 + pl.ngroups - 1) / pl.ngroups;
#pragma unroll 1
  for (int r = 4 + l16; r < niter; r += 16) {
    const int j = a.p0 + r * pl.ngroups + pl.gi;
    if (j < a.p1 && j != a.L - 1) {
      const int slot = (j >> psh) - (a.p0 >> psh);
      const int pg = (pgs != nullptr && slot < 16) ? pgs[slot] : __ldcg(c.p.kv_indices + a.kv_base + (j >> psh));
      const size_t src = ((((size_t)pg << psh) + (j & pmask)) * pl.HKV + a.h) * kHeadDim;
      const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(op.k_cache) + src;
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(op.v_cache) + src;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(kp));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(kp + 64));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(vp));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(vp + 64));
    }
  }
}

// Prompt chunks (several tokens of one request in an iteration).  Waits for the op's barrier, then one
// warp per (token, kv head) pair normalises and rotates the token's new K and stores it, with its V, at
// the token's own position in the cache; a second grid barrier makes all of them visible.  Returns true
// when the launch is aborting.  (Both halves of a warp compute the same pair: the shuffles in
// head_norm_rope use the full mask.)
__device__ __noinline__ bool attn_barrier_then_append(Ctx& c, const OpDesc& op, const AttnPlan& pl, const int* lens, int T) {
  const KParams& p = c.p;
  if (op.flags & F_SYNC_BEFORE) {
    grid_wait(c);
    if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
    c.dead = c.flags()[3] != 0;
    if (c.dead) return true;
  } else if (op.flags & F_LL_IN) {
    // no barrier stands before this op, but a prompt chunk reads the plain rows of every token: a full one here
    grid_sync(c);
    if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
    c.dead = c.flags()[3] != 0;
    if (c.dead) return true;
  } else if (op_barrier(c, op)) {
    return true;
  }
  const int l16 = c.lane & 15;
  const bool dbl_k = op.aux0 < 32;
  const uint4 wk = __ldg(reinterpret_cast<const uint4*>(op.k_norm_w) + l16);
#pragma unroll 1
  for (int pair = blockIdx.x * kNumConsumerWarps + c.warp; pair < T * pl.HKV; pair += gridDim.x * kNumConsumerWarps) {
    const int t = pair / pl.HKV, h = pair % pl.HKV;
    const int L = lens[t];
    if (L <= 0) continue;
    const int pos = min(L - 1, op.aux2 - 1);
    const uint4 cs = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.cos) + (size_t)pos * kHeadDim) + l16);
    const uint4 sn = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.sin) + (size_t)pos * kHeadDim) + l16);
    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)t * op.ld_in + (size_t)h * (pl.qpk + 2) * kHeadDim;
    const uint4 vnew = __ldcg(reinterpret_cast<const uint4*>(row + (pl.qpk + 1) * kHeadDim) + l16);
    F8 kf;
    unpack8(__ldcg(reinterpret_cast<const uint4*>(row + pl.qpk * kHeadDim) + l16), kf.v);
    kf = head_norm_rope(kf, wk, cs, sn, l16, op.flags, p.numerics, dbl_k);
    const int pg = __ldcg(p.kv_indices + lens[kAttnLensMax + t] + ((L - 1) >> p.page_shift));
    if (c.lane < 16) {
      const size_t dst = ((((size_t)pg << p.page_shift) + ((L - 1) & (p.page_size - 1))) * pl.HKV + h) * kHeadDim;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.k_cache) + dst)[l16] = pack8(kf.v);
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.v_cache) + dst)[l16] = vnew;
    }
  }
  grid_sync(c);
  c.dead = c.flags()[3] != 0;
  return c.dead;
}

// Larger batches: with more (request, kv head) pairs than CTAs and sequences short enough to
// need no split, a CTA runs 2 or 4 pairs side by side instead of one after the other: its 8
// warps form groups of 4 or 2, every group is a small copy of the CTA-wide scheme (its warps
// split the positions, a half-warp serves all q heads of the pair, the group meets on a
// named barrier of its own).  The fixed latencies of a pair (q path, row fetches, combine)
// are then paid once per round of `groups` pairs.
__device__ __forceinline__ void group_sync(int g, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(2 + g), "r"(nthreads) : "memory");
}
__device__ __noinline__ void attention_groups(Ctx& c, const OpDesc& op, const AttnPlan& pl0, const int* lens, int wpg, int T, bool chunked) {
  const KParams& p = c.p;
  const int G = gridDim.x;
  AttnPlan pl = pl0;
  const int ngrp = kNumConsumerWarps / wpg;
  const int g = c.warp / wpg, lw = c.warp % wpg;
  const int gthreads = wpg * 32, gtid = lw * 32 + c.lane;
  const int l16 = c.lane & 15;
  const int hq = pl.qpk;  // at most 4 here
  pl.ngroups = 2 * wpg;
  pl.gi = 2 * lw + (c.lane >> 4);
  const float sc = 1.4426950408889634f * 0.08838834764831845f;  // log2(e) / sqrt(128)
  const bool dbl_q = op.aux1 < 32, dbl_k = op.aux0 < 32;
  // per group: q heads [4][16] + new k [16] (bf16 x 8 per entry); per warp: 4 heads x 128 floats, (max, sum) x 4
  uint4* sm_q = reinterpret_cast<uint4*>(c.smem + p.x_off) + g * 80;
  uint4* sm_k = sm_q + 64;
  float* sm_o = reinterpret_cast<float*>(reinterpret_cast<uint4*>(c.smem + p.x_off) + 4 * 80) + c.warp * 4 * kHeadDim;
  float* sm_ml = reinterpret_cast<float*>(reinterpret_cast<uint4*>(c.smem + p.x_off) + 4 * 80) + kNumConsumerWarps * 4 * kHeadDim;
  bool first = true;
  if (chunked) {
    if (attn_barrier_then_append(c, op, pl, lens, T)) return;
    first = false;
  }
#pragma unroll 1
  for (int task = blockIdx.x + G * g;; task += G * ngrp) {
    AttnTask a;
    attn_prepare(c, op, pl, lens, task, l16, a);
    if (first) {
      first = false;
      if (op.flags & F_SYNC_BEFORE) {  // op_barrier with the wait inlined: the prefetched rows stay in registers
        grid_wait(c);
        if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
        c.dead = c.flags()[3] != 0;
        if (c.dead) return;
      } else if (op_barrier(c, op)) {
        return;
      }
    }
    if (task >= pl.ntasks) break;   // uniform within the group
    if (!a.valid) continue;
    const int L = a.L;
    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)a.t * op.ld_in +
                               (size_t)a.h * (pl.qpk + 2) * kHeadDim;
    const uint4 vnew = __ldcg(reinterpret_cast<const uint4*>(row + (pl.qpk + 1) * kHeadDim) + l16);
#pragma unroll 1
    for (int h = lw; h < hq; h += wpg) {  // this warp's share of the q heads
      F8 q;
      unpack8(__ldcg(reinterpret_cast<const uint4*>(row + h * kHeadDim) + l16), q.v);
      q = head_norm_rope(q, a.wq, a.cs, a.sn, l16, op.flags, p.numerics, dbl_q);
      if (c.lane < 16) sm_q[h * 16 + l16] = pack8(q.v);
    }
    if (lw == wpg - 1) {  // the group's last warp also prepares the new k
      F8 kf;
      unpack8(__ldcg(reinterpret_cast<const uint4*>(row + pl.qpk * kHeadDim) + l16), kf.v);
      kf = head_norm_rope(kf, a.wk, a.cs, a.sn, l16, op.flags, p.numerics, dbl_k);
      const uint4 kn = pack8(kf.v);
      if (c.lane < 16) {
        sm_k[l16] = kn;
        if (a.p1 == L && !chunked) {  // append the new token's K and V to the cache
          const size_t dst = ((((size_t)a.new_page << p.page_shift) + ((L - 1) & (p.page_size - 1))) * pl.HKV + a.h) * kHeadDim;
          reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.k_cache) + dst)[l16] = kn;
          reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.v_cache) + dst)[l16] = vnew;
        }
      }
    }
    group_sync(g, gthreads);
    uint4 qv[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) qv[h] = (h < hq) ? sm_q[h * 16 + l16] : make_uint4(0, 0, 0, 0);
    const uint4 knew = sm_k[l16];
    float m[4], l[4], o[4][8];
    attn_rows(c, op, pl, a, l16, hq, qv, knew, vnew, sc, m, l, o);
    // the two halves of a warp by shuffle, then the group's warps through shared memory
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      if (h < hq) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m[h], 16), l2 = __shfl_xor_sync(0xffffffffu, l[h], 16);
        const float M = fmaxf(m[h], m2);
        const float f1 = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - M), f2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - M);
        const float lsum = f1 * l[h] + f2 * l2;
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = f1 * o[h][i] + f2 * __shfl_xor_sync(0xffffffffu, o[h][i], 16);
        if (c.lane < 16) {
          float* dst = sm_o + h * kHeadDim + l16 * 8;
          reinterpret_cast<float4*>(dst)[0] = make_float4(r[0], r[1], r[2], r[3]);
          reinterpret_cast<float4*>(dst)[1] = make_float4(r[4], r[5], r[6], r[7]);
          if (l16 == 0) {
            sm_ml[(c.warp * 4 + h) * 2] = M;
            sm_ml[(c.warp * 4 + h) * 2 + 1] = lsum;
          }
        }
      }
    }
    group_sync(g, gthreads);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)a.t * op.ld_out +
                         (size_t)a.h * pl.qpk * kHeadDim;
    const float* go = reinterpret_cast<const float*>(reinterpret_cast<const uint4*>(c.smem + p.x_off) + 4 * 80) +
                      (size_t)(g * wpg) * 4 * kHeadDim;  // the group's first warp slot
#pragma unroll 1
    for (int e = gtid; e < hq * kHeadDim; e += gthreads) {
      const int h = e >> 7, d = e & 127;
      float M = -INFINITY;
      for (int w = 0; w < wpg; ++w) M = fmaxf(M, sm_ml[((g * wpg + w) * 4 + h) * 2]);
      float Ls = 0.f, O = 0.f;
      for (int w = 0; w < wpg; ++w) {
        const float mw = sm_ml[((g * wpg + w) * 4 + h) * 2];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        Ls += f * sm_ml[((g * wpg + w) * 4 + h) * 2 + 1];
        O += f * go[(w * 4 + h) * kHeadDim + d];
      }
      out[e] = __float2bfloat16_rn(__fdividef(O, Ls));
    }
    group_sync(g, gthreads);  // the group's buffers are free again
  }
}

// aux0 = kv heads, aux1 = q heads (q heads per kv head: 1, 2, 4 or 8).  Tokens: one per
// request, token t == request slot t.
// The pass of a task over its positions on the tensor cores (wider batches; up to four q heads per kv head).
// One warp takes 16 positions at a time (tiles warp, warp + 8, ... of the task's range) for all q heads:
//   S = Q K^T   mma.m16n8k16, M = the q heads (rows 4..15 are padding), N = 8 positions, K = 128 dims in 8 steps
//   O += P V    M = the q heads, K = 16 positions, N = 128 dims in 16 tiles of 8
// with the fragments loaded STRAIGHT from the cache rows, no shared-memory staging and no ldmatrix: a dot
// product does not care in which order the dims are walked, so k step s of lane j of a quad stands for dims
// 32 (s / 2) + 8 j + 4 (s % 2) + {0..3} (the quad reads 64 contiguous bytes of the K row of position lane / 4
// per load), and output column n of tile t stands for dim 64 (t / 8) + 8 n + t % 8 (eight lanes read 128
// contiguous bytes of a V row per load; two rows are paired up per register with byte permutes).  The scalar pass (attn_rows1) issued about twenty times the instructions per position.
// Leaves (max, sum, output) of slot warp * qpk + head in shared memory for the combine.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// (rows 8..15 of the M side are padding: their two accumulators are scratch registers shared by all tiles)
__device__ __forceinline__ void mma_bf16_top(float& c0, float& c1, float& z0, float& z1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1)
               : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __noinline__ void attn_tc_rows(const Ctx& c, const OpDesc& op, const AttnPlan& pl, const AttnTask& a, const uint4* sm_q,
                                          const uint4* sm_knew, const uint4* sm_vnew, float sc, float* sm_o, float* sm_m,
                                          float* sm_l, const int* pgt, bool subst_new) {
  const int lane = c.lane, g = lane >> 2, j = lane & 3;
  const int psh = c.p.page_shift, pmask = c.p.page_size - 1;
  const bool hv = g < pl.qpk;
  uint32_t qa0[8], qa2[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const uint2 v = hv ? *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(sm_q) + g * 256 + (32 * (s >> 1) + 8 * j + 4 * (s & 1)) * 2)
                       : make_uint2(0u, 0u);
    qa0[s] = v.x;
    qa2[s] = v.y;
  }
  float m = -INFINITY, l = 0.f;
  float oacc[16][2], z0 = 0.f, z1 = 0.f;
#pragma unroll
  for (int t = 0; t < 16; ++t) oacc[t][0] = oacc[t][1] = 0.f;
  const int base_slot = a.p0 >> psh;
  const int ntiles = (a.p1 - a.p0 + 15) >> 4;
  const char* kc = reinterpret_cast<const char*>(op.k_cache);
  const char* vc = reinterpret_cast<const char*>(op.v_cache);
#pragma unroll 1
  for (int ti = c.warp; ti < ntiles; ti += kNumConsumerWarps) {
    const int pos0 = a.p0 + 16 * ti;
    // K: positions pos0 + g and pos0 + 8 + g, dims [32 j, 32 j + 32)
    uint4 kr[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int pos = pos0 + 8 * u + g;
#pragma unroll
      for (int i = 0; i < 4; ++i) kr[u][i] = make_uint4(0u, 0u, 0u, 0u);
      if (pos < a.p1) {
        if (subst_new && pos == a.L - 1) {
#pragma unroll
          for (int i = 0; i < 4; ++i) kr[u][i] = sm_knew[4 * i + j];
        } else {
          const int slot = (pos >> psh) - base_slot;
          const int pg = slot < 32 ? pgt[slot] : __ldcg(c.p.kv_indices + a.kv_base + (pos >> psh));
          const uint4* src = reinterpret_cast<const uint4*>(kc + ((((size_t)pg << psh) + (pos & pmask)) * pl.HKV + a.h) * (kHeadDim * 2)) + j;
#pragma unroll
          for (int i = 0; i < 4; ++i) kr[u][i] = __ldcg(src + 4 * i);  // a quad reads 64 contiguous bytes per load
        }
      }
    }
    // V: positions pos0 + 2 j + {0, 1} and pos0 + 8 + 2 j + {0, 1}, dims [16 g, 16 g + 16)
    uint4 vr[4][2];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int pos = pos0 + 2 * j + (r & 1) + 8 * (r >> 1);
      vr[r][0] = vr[r][1] = make_uint4(0u, 0u, 0u, 0u);
      if (pos < a.p1) {
        if (subst_new && pos == a.L - 1) {
          vr[r][0] = sm_vnew[g];
          vr[r][1] = sm_vnew[8 + g];
        } else {
          const int slot = (pos >> psh) - base_slot;
          const int pg = slot < 32 ? pgt[slot] : __ldcg(c.p.kv_indices + a.kv_base + (pos >> psh));
          const uint4* src = reinterpret_cast<const uint4*>(vc + ((((size_t)pg << psh) + (pos & pmask)) * pl.HKV + a.h) * (kHeadDim * 2)) + g;
          vr[r][0] = __ldcg(src);  // the eight lanes with this j read 128 contiguous bytes per load
          vr[r][1] = __ldcg(src + 8);
        }
      }
    }
    // S = Q K^T for the two groups of 8 positions
    float sv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const uint4& k0 = kr[0][s >> 1];
      const uint4& k1 = kr[1][s >> 1];
      mma_bf16_top(sv[0], sv[1], z0, z1, qa0[s], qa2[s], (s & 1) ? k0.z : k0.x, (s & 1) ? k0.w : k0.y);
      mma_bf16_top(sv[2], sv[3], z0, z1, qa0[s], qa2[s], (s & 1) ? k1.z : k1.x, (s & 1) ? k1.w : k1.y);
    }
    // this lane: head g at positions pos0 + 2 j + {0, 1} (sv[0], sv[1]) and pos0 + 8 + 2 j + {0, 1} (sv[2], sv[3])
    float tmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int pos = pos0 + 2 * j + (i & 1) + 8 * (i >> 1);
      sv[i] = pos < a.p1 ? sv[i] * sc : -INFINITY;
      tmax = fmaxf(tmax, sv[i]);
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float mn = fmaxf(m, tmax);  // finite: the tile holds at least one position of the range
    const float alpha = exp2f(m - mn);
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = exp2f(sv[i] - mn);
    l = l * alpha + ((pr[0] + pr[1]) + (pr[2] + pr[3]));  // this lane's share of the row sum: the quad adds up at the end
    m = mn;
    const uint32_t pa0 = pack2(pr[0], pr[1]), pa2 = pack2(pr[2], pr[3]);
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      oacc[t][0] *= alpha;
      oacc[t][1] *= alpha;
      // dim 16 g + t of the four V rows: element t of the lane's 16, two rows per register
      const uint4& a0 = vr[0][t >> 3];
      const uint4& a1 = vr[1][t >> 3];
      const uint4& a2 = vr[2][t >> 3];
      const uint4& a3 = vr[3][t >> 3];
      const int w = (t >> 1) & 3;
      const uint32_t w0 = w == 0 ? a0.x : (w == 1 ? a0.y : (w == 2 ? a0.z : a0.w));
      const uint32_t w1 = w == 0 ? a1.x : (w == 1 ? a1.y : (w == 2 ? a1.z : a1.w));
      const uint32_t w2 = w == 0 ? a2.x : (w == 1 ? a2.y : (w == 2 ? a2.z : a2.w));
      const uint32_t w3 = w == 0 ? a3.x : (w == 1 ? a3.y : (w == 2 ? a3.z : a3.w));
      const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
      mma_bf16_top(oacc[t][0], oacc[t][1], z0, z1, pa0, pa2, prmt(w0, w1, sel), prmt(w2, w3, sel));
    }
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (hv) {
    const int w = c.warp * pl.qpk + g;
    if (j == 0) {
      sm_m[w] = m;
      sm_l[w] = l;
    }
    float* dst = sm_o + w * kHeadDim + 16 * j;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      dst[64 * (t >> 3) + (t & 7)] = oacc[t][0];
      dst[64 * (t >> 3) + 8 + (t & 7)] = oacc[t][1];
    }
  }
}

template <int PATH>
__device__ __noinline__ void op_attention(Ctx& c, const OpDesc& op, int T) {
  const KParams& p = c.p;
  const int G = gridDim.x;
  MK_STAMP(c, 0);
  if (p.debug_flags & 2) {  // measurement aid: the op keeps its barrier and does nothing else
    op_barrier(c, op);
    return;
  }
  // arrive at the op's barrier first: everything up to the wait below is independent of other CTAs
  if (op.flags & F_SYNC_BEFORE) grid_arrive(c);
  // Per-iteration cache in the scratch region (nothing else touches these bytes): sequence
  // lengths incl. the new token [128], page-table offsets [128], then per half-warp the page
  // numbers of its first four rows and of the new token [16][8].  The metadata only changes
  // between iterations, so the first attention op of an iteration fills it and the other
  // layers start their K/V row loads without any dependent look-up.
  int* lens = reinterpret_cast<int*>(c.red() + 64);
  int* pgc = lens + 2 * kAttnLensMax + (c.tid >> 4) * 8;
  int* pgs = lens + 2 * kAttnLensMax + 16 * 8;  // [16]: page numbers of the first task's chunk, from its first page on
  const int key = (c.iter << 8) ^ (op.aux0 * 16 + op.aux1);  // iteration and head geometry
  const bool fill = c.attn_iter != key;
  c.attn_iter = key;
  int* multi = pgs + 16 + 3 + 9;  // [1]: some request has several tokens in this iteration (a prompt chunk)
  if (fill) {
    if (c.tid == 0) *multi = 0;
    consumer_sync();
    // Token t of request r (qo_indptr[r] <= t < qo_indptr[r + 1]) sits at position kv_len(r) - (tokens of r behind
    // it) - 1: its sequence length, itself included, is what the tasks below call L.
#pragma unroll 1
    for (int r = c.tid; r < p.max_reqs; r += kNumConsumers) {
      const int q0 = __ldcg(p.qo_indptr + r), q1 = min(__ldcg(p.qo_indptr + r + 1), T);
      if (q1 > q0) {
        const int first = __ldcg(p.kv_indptr + r), last = __ldcg(p.kv_indptr + r + 1);
        const int kvlen = (last - first - 1) * p.page_size + __ldcg(p.kv_last_page_len + r);
        for (int t = q0; t < q1; ++t) {
          lens[t] = kvlen - (q1 - 1 - t);
          lens[kAttnLensMax + t] = first;
        }
        if (q1 - q0 > 1) *multi = 1;
      }
    }
    consumer_sync();
  }
  AttnPlan pl;
  pl.HKV = op.aux0;
  pl.qpk = op.aux1 / op.aux0;
  int* plan = pgs + 16;   // [0] chunk size, [1] chunks of the longest request, [2] tasks: the same in every layer of an iteration
  int* geom = plan + 3;   // [9]: the CTA's first task, see attn_prepare
  bool all_short;         // no sequence of the iteration is longer than 256 tokens (bit 8 of plan[1])
  if (fill) {
    int Lmax = 1;
#pragma unroll 1
    for (int r = 0; r < T; ++r) Lmax = max(Lmax, lens[r]);
    const int nb_max = (Lmax + 15) >> 4;
    int bpc = (T * pl.HKV * nb_max + G - 1) / G;  // 16-position blocks per chunk: one round of tasks
    bpc = max(bpc, (nb_max + p.attn_max_chunks - 1) / p.attn_max_chunks);
    bpc = max(bpc, 1);
    // one round of tasks: a chunk count that leaves a few CTAs a second task doubles the op's time
    while (T * pl.HKV <= G && T * pl.HKV * ((nb_max + bpc - 1) / bpc) > G) ++bpc;
    pl.CS = bpc * 16;
    pl.nch_max = (nb_max + bpc - 1) / bpc;
    pl.ntasks = T * pl.HKV * pl.nch_max;
    all_short = Lmax <= 256;
    if (c.tid == 0) {
      plan[0] = pl.CS;
      plan[1] = pl.nch_max | (all_short ? 256 : 0);
      plan[2] = pl.ntasks;
    }
  } else {
    pl.CS = plan[0];
    pl.nch_max = plan[1] & 255;
    all_short = (plan[1] & 256) != 0;
    pl.ntasks = plan[2];
  }
  // More (request, kv head) pairs than CTAs, all of them short: several pairs side by side per CTA (the fixed
  // cost of a pair, about 12 us, dominates; measured at 64 requests of 100 tokens: 48 us against 68 us one
  // pair at a time).
  if constexpr (PATH == PATH_UMMA) {
    if (pl.nch_max == 1 && pl.ntasks > G && pl.qpk <= 4 && all_short) {
      attention_groups(c, op, pl, lens, pl.ntasks > 2 * G ? 2 : 4, T, *multi != 0);
      return;
    }
  }
  // wider batches: the pass over the positions runs on the tensor cores (up to four q heads per kv head; measured
  // at 16 requests: 20 us against 24 us at 100 tokens, 33 us against 83 us at 600; slower below 9 batched tokens)
  const bool tc = PATH != PATH_ROWS && pl.qpk <= 4 && p.x_rows >= 16;
  const int l16 = c.lane & 15;
  // Half-warp hw serves q head (hw % qpk) of the kv-head group for the positions of group
  // (hw / qpk): one head per thread keeps the row loop and the combine small (this code runs
  // once per layer out of a cold instruction cache), and the two halves of a warp read the
  // same K/V rows, so their loads share a request.
  const int hw = 2 * c.warp + (c.lane >> 4);
  const int head = hw % pl.qpk;
  pl.ngroups = tc ? kNumConsumerWarps : 16 / pl.qpk;  // slots per head in the combine: warps, or half-warp groups
  pl.gi = hw / pl.qpk;
  const int part_stride = pl.qpk * (kHeadDim + 2);
  const float sc = 1.4426950408889634f * 0.08838834764831845f;  // log2(e) / sqrt(128)
  uint4* sm_q = reinterpret_cast<uint4*>(c.smem + p.x_off);     // [8 heads][16 lanes]: q after norm and RoPE
  uint4* sm_k = sm_q + 8 * 16;                                  // [16 lanes]: the new k
  uint4* sm_v = sm_k + 16;                                      // [16 lanes]: the new v (tensor-core pass)
  const int nslots = tc ? kNumConsumerWarps * pl.qpk : 16;
  float* sm_o = reinterpret_cast<float*>(sm_v + 16);            // [slots][128]: 16 half-warps, or warp x head
  float* sm_m = sm_o + nslots * kHeadDim;                       // [slots]
  float* sm_l = sm_m + nslots;
  int* pgt = reinterpret_cast<int*>(sm_l + nslots);             // [32]: page numbers of the task's range (tensor-core pass)
  const bool dbl_q = op.aux1 < 32, dbl_k = op.aux0 < 32;
  const int kw = pl.qpk & 7;  // the warp that prepares the new k (warp 0 when all eight prepare q heads)

  bool first = true;
  const bool chunked = *multi != 0;
  if (chunked) {
    // A prompt chunk: its tokens attend to each other's K/V, which only exist once every token's K has been
    // normalised, rotated and appended.  So this iteration appends first, for all tokens, behind the op's
    // own barrier, and meets at one more grid barrier before any row is read (nothing is fetched early).
    if (attn_barrier_then_append(c, op, pl, lens, T)) return;
    first = false;
  }
#pragma unroll 1
  for (int task = blockIdx.x;; task += G) {
    AttnTask a;
    if constexpr (PATH == PATH_ROWS)
      attn_prepare<false>(c, op, pl, lens, task, l16, a, (first && !chunked) ? pgc : nullptr, fill, (first && !chunked) ? geom : nullptr);
    else
      attn_prepare<false, false>(c, op, pl, lens, task, l16, a, nullptr, true, nullptr);
    if (first) {
      // everything above is independent of this layer's QKV rows: fetched ahead of the barrier
      first = false;
      if (a.valid) {
        if (fill && c.tid < 16) {  // (read only after the barrier's CTA-wide sync)
          const int slot = (a.p0 >> p.page_shift) + c.tid;
          if ((slot << p.page_shift) < a.p1) pgs[c.tid] = __ldcg(p.kv_indices + a.kv_base + slot);
        }
        if constexpr (PATH == PATH_ROWS) attn_l2_ahead(c, op, pl, a, l16, fill ? nullptr : pgs);
      }
      MK_STAMP(c, 1);
      if (op.flags & F_SYNC_BEFORE) {  // op_barrier, with the wait inlined
        grid_wait(c);
        if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
        c.dead = c.flags()[3] != 0;
        if (c.dead) return;
      } else if (op.flags & F_LL_IN) {
        // (no look at the abort flag: the polls of the tagged input watch it)
        consumer_sync();
        if (c.pr != nullptr && c.tid == 0) c.pr[1] = globaltimer();
      } else if (op_barrier(c, op)) {
        return;
      }
    }
    if (task >= pl.ntasks) break;
    if (!a.valid) continue;
    const int L = a.L;
    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)a.t * op.ld_in +
                               (size_t)a.h * (pl.qpk + 2) * kHeadDim;
    // tagged input: the task polls the words of its own kv-head group only (a prompt chunk has had its barrier)
    const bool ll_in = (op.flags & F_LL_IN) && !chunked;
    const uint2* llr = ll_row(op.ll_in, op.ld_in, a.t) + ((a.h * (pl.qpk + 2) * kHeadDim) >> 1);
    const unsigned tag_in = ll_tag_of(c, op.ll_in_op);
    const bool do_q = c.warp < pl.qpk, do_k = c.warp == kw;
    uint4 vnew, xq = make_uint4(0, 0, 0, 0), xk = make_uint4(0, 0, 0, 0);
    // norm weights and the cos/sin row of the position, for the warps that prepare a head
    uint4 nw = make_uint4(0, 0, 0, 0), ncs = nw, nsn = nw;
    if (do_q || do_k) {
      const int pos = min(L - 1, op.aux2 - 1);  // aux2 = rows of the cos/sin tables
      nw = __ldg(reinterpret_cast<const uint4*>(do_q ? op.q_norm_w : op.k_norm_w) + l16);
      ncs = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.cos) + (size_t)pos * kHeadDim) + l16);
      nsn = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.sin) + (size_t)pos * kHeadDim) + l16);
    }
    if (ll_in) {  // all loads first, then whatever has not arrived is polled
      const uint4* sv = reinterpret_cast<const uint4*>(llr + (((pl.qpk + 1) * kHeadDim + l16 * 8) >> 1));
      const uint4* sq = reinterpret_cast<const uint4*>(llr + ((c.warp * kHeadDim + l16 * 8) >> 1));
      const uint4* sk = reinterpret_cast<const uint4*>(llr + ((pl.qpk * kHeadDim + l16 * 8) >> 1));
      const uint4 v0 = ld_gpu_v4(sv), v1 = ld_gpu_v4(sv + 1);
      uint4 q0 = v0, q1 = v1, k0 = v0, k1 = v1;
      if (do_q) {
        q0 = ld_gpu_v4(sq);
        q1 = ld_gpu_v4(sq + 1);
      }
      if (do_k) {
        k0 = ld_gpu_v4(sk);
        k1 = ld_gpu_v4(sk + 1);
      }
      vnew = ll_take8(c, sv, v0, v1, tag_in);
      if (do_q) xq = ll_take8(c, sq, q0, q1, tag_in);
      if (do_k) xk = ll_take8(c, sk, k0, k1, tag_in);
    } else {
      vnew = __ldcg(reinterpret_cast<const uint4*>(row + (pl.qpk + 1) * kHeadDim) + l16);
      if (do_q) xq = __ldcg(reinterpret_cast<const uint4*>(row + c.warp * kHeadDim) + l16);
      if (do_k) xk = __ldcg(reinterpret_cast<const uint4*>(row + pl.qpk * kHeadDim) + l16);
    }
    // norm + RoPE once per CTA: warp w < qpk prepares q head w, one warp the new k
    if (do_q) {
      F8 q;
      unpack8(xq, q.v);
      q = head_norm_rope(q, nw, ncs, nsn, l16, op.flags, p.numerics, dbl_q);
      if (c.lane < 16) sm_q[c.warp * 16 + l16] = pack8(q.v);  // exact: the values are bf16 already
    }
    if (do_k) {
      F8 kf;
      unpack8(xk, kf.v);
      kf = head_norm_rope(kf, do_q ? __ldg(reinterpret_cast<const uint4*>(op.k_norm_w) + l16) : nw, ncs, nsn, l16, op.flags, p.numerics, dbl_k);
      const uint4 kn = pack8(kf.v);
      if (c.lane < 16) {
        sm_k[l16] = kn;
        sm_v[l16] = vnew;
        if (a.p1 == L && !chunked) {  // the last chunk appends the new token's K and V to the cache
          const size_t dst = ((((size_t)a.new_page << p.page_shift) + ((L - 1) & (p.page_size - 1))) * pl.HKV + a.h) * kHeadDim;
          reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.k_cache) + dst)[l16] = kn;
          reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.v_cache) + dst)[l16] = vnew;
        }
      }
    }
    if (PATH != PATH_ROWS && tc && c.tid < 32) {  // the page numbers of the task's range, for the tensor-core pass
      const int slot = (a.p0 >> p.page_shift) + c.tid;
      if ((slot << p.page_shift) < a.p1) pgt[c.tid] = __ldcg(p.kv_indices + a.kv_base + slot);
    }
    consumer_sync();
    MK_STAMP(c, 2);
    bool done_rows = false;
    if constexpr (PATH != PATH_ROWS) {
      if (tc) {
        attn_tc_rows(c, op, pl, a, sm_q, sm_k, sm_v, sc, sm_o, sm_m, sm_l, pgt, !chunked);
        done_rows = true;
      }
    }
    if (!done_rows) {
      const uint4 qv = sm_q[head * 16 + l16];
      const uint4 knew = sm_k[l16];
      float m, l, o[8];
      if constexpr (PATH != PATH_ROWS) attn_fetch_rows(c, op, pl, a, 0, l16, a.kr, a.vr);  // (nothing was fetched ahead)
      attn_rows1(c, op, pl, a, l16, qv, knew, vnew, sc, m, l, o, (task == (int)blockIdx.x && !chunked) ? pgs : nullptr);
      // every half-warp leaves its (max, sum, output) in shared memory; one pass over the output
      // elements then combines the position groups of each head
      float* dst = sm_o + hw * kHeadDim + l16 * 8;
      reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
      if (l16 == 0) {
        sm_m[hw] = m;
        sm_l[hw] = l;
      }
    }
    MK_STAMP(c, 3);
    consumer_sync();
    float* part = p.attn_part + (((size_t)a.t * pl.HKV + a.h) * p.attn_max_chunks + a.ch) * part_stride;
    // tagged partials (see attn_merge_ll) when the op's output is tagged and the host gave them room
    const bool ll_part = (op.flags & F_LL_OUT) && p.attn_part_ll != nullptr;
    uint2* partw = p.attn_part_ll + (((size_t)a.t * pl.HKV + a.h) * p.attn_max_chunks + a.ch) * part_stride;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)a.t * op.ld_out +
                         (size_t)a.h * pl.qpk * kHeadDim;
    uint2* ll_out = (op.flags & F_LL_OUT) ? reinterpret_cast<uint2*>(op.ll_out) + (size_t)a.t * (size_t)(op.ld_out >> 1) +
                                                ((a.h * pl.qpk * kHeadDim) >> 1)
                                          : nullptr;
#pragma unroll 1
    for (int e = c.tid; e < pl.qpk * kHeadDim; e += kNumConsumers) {
      const int eh = e >> 7, d = e & 127;
      float M = -INFINITY;
#pragma unroll 4
      for (int g = 0; g < pl.ngroups; ++g) M = fmaxf(M, sm_m[g * pl.qpk + eh]);
      float Ls = 0.f, O = 0.f;
#pragma unroll 4  // (four reads of shared memory in flight: 0.5 % of a batch-1 step against the rolled loop)
      for (int g = 0; g < pl.ngroups; ++g) {
        const int w = g * pl.qpk + eh;
        const float mw = sm_m[w];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        Ls += f * sm_l[w];
        O += f * sm_o[w * kHeadDim + d];
      }
      if (a.nch == 1) {
        const __nv_bfloat16 y = __float2bfloat16_rn(__fdividef(O, Ls));
        out[e] = y;
        if (op.flags & F_LL_OUT) {  // (whole warps run this loop: its bound is a multiple of 128)
          const uint32_t lo = (uint32_t)__bfloat16_as_ushort(y);
          const uint32_t hi = __shfl_down_sync(0xffffffffu, lo, 1);
          if (!(e & 1)) st_gpu_v2(ll_out + (e >> 1), lo | (hi << 16), ll_tag_of(c, c.cur_op));
        }
      } else if (ll_part) {
        st_gpu_v2(partw + e, __float_as_uint(O), ll_tag_of(c, c.cur_op));
        if (d == 0) {
          st_gpu_v2(partw + pl.qpk * kHeadDim + eh, __float_as_uint(M), ll_tag_of(c, c.cur_op));
          st_gpu_v2(partw + pl.qpk * kHeadDim + pl.qpk + eh, __float_as_uint(Ls), ll_tag_of(c, c.cur_op));
        }
      } else {
        part[e] = O;
        if (d == 0) {
          part[pl.qpk * kHeadDim + eh] = M;
          part[pl.qpk * kHeadDim + pl.qpk + eh] = Ls;
        }
      }
    }
    MK_STAMP(c, 4);
    if (a.nch > 1 && ll_part) {
      attn_merge_ll(c, partw - (size_t)a.ch * part_stride, out, ll_out, a.nch, a.ch, pl.qpk, part_stride, ll_tag_of(c, c.cur_op));
    } else if (a.nch > 1) {
      consumer_sync();  // the CTA's partial is complete; thread 0's release below publishes all of it
      MK_STAMP(c, 5);
      volatile int* fl = c.flags();
      unsigned* cnt = p.attn_count + (size_t)a.t * pl.HKV + a.h;
      const float* base = p.attn_part + (((size_t)a.t * pl.HKV + a.h) * p.attn_max_chunks) * part_stride;
      if (c.tid == 0) {
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(cnt) : "memory");
        fl[2] = (old == (unsigned)(a.nch - 1)) ? 1 : 0;
      }
      consumer_sync();
      MK_STAMP(c, 6);
      // The chunk that arrives last merges all of them.  (A fixed merger per kv head, polling the
      // counter, measured slower: the last arriver knows at once that it is the last.)
      if (fl[2] != 0) {
        attn_merge(c, base, out, a.nch, pl.qpk, part_stride, ll_out, ll_tag_of(c, c.cur_op));
        if (c.tid == 0) *cnt = 0u;
      }
    }
    consumer_sync();
    MK_STAMP(c, 7);
  }
}

// ------------------------------------------------------------------------------------
// small ops
// ------------------------------------------------------------------------------------
// aux0 = embedding rows
__device__ void op_embed(Ctx& c, const OpDesc& op, int T) {
  const int nseg = (op.n + 2047) / 2048;
  const long long* ids = reinterpret_cast<const long long*>(op.in);
  for (int u = blockIdx.x; u < T * nseg; u += gridDim.x) {
    const int tok = u / nseg, seg = u % nseg;
    long long id = __ldcg(ids + (size_t)tok * op.ld_in);
    if (id < 0 || id >= op.aux0) {
      if (c.tid == 0) raise_abort(c, ST_BAD_TOKEN, tok, (int)id);
      id = 0;
    }
    const int col = seg * 2048 + c.tid * 8;
    if (col < op.n) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.w) + (size_t)id * op.ld_res + col));
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)tok * op.ld_out + col) = v;
    }
  }
}

__device__ void op_rmsnorm(Ctx& c, const OpDesc& op, int T) {
  const int kp = ((op.n + 63) / 64) * 64;
  // the norm weights do not depend on other CTAs: a CTA that has a row fetches them ahead of the barrier
  uint4 pre_w[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  const bool pre = (kp >> 3) <= 4 * kNumConsumers;
  if (pre && (int)blockIdx.x < T) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = c.tid + kNumConsumers * i;
      if (v < (op.n >> 3)) pre_w[i] = __ldg(reinterpret_cast<const uint4*>(op.w) + v);
    }
  }
  if (op_barrier(c, op)) return;
  for (int tok = blockIdx.x; tok < T; tok += gridDim.x) {
    // (the sums are also stored into the gathered tensor's own rows when the host asked for it: aux0)
    if (MK_XF(op, F_GATHER_IN)) stage_x(c, nullptr, op.ld_in, op.n, kp, op.w, tok, 1, tok + 1, pre ? pre_w : nullptr, true,
                                         (op.aux0 && pre) ? const_cast<void*>(op.in) : nullptr);
    else stage_x(c, reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)tok * op.ld_in, op.ld_in, op.n, kp, op.w, 0, 1, 1,
                 pre ? pre_w : nullptr);
    const uint4* xs = reinterpret_cast<const uint4*>(c.smem + c.p.x_off);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)tok * op.ld_out);
    for (int v = c.tid; v < (op.n >> 3); v += kNumConsumers) dst[v] = xs[v];
    consumer_sync();
  }
}

// aux0 = columns per [gate | up] block of the input
__device__ void op_silu_mul(Ctx& c, const OpDesc& op, int T) {
  const int bk = op.aux0;
  const int nvec = op.n >> 3;
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(op.in);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  const long long rows = (long long)T * (op.aux1 > 0 ? op.aux1 : 1);  // aux1: rows per token (expert slots of a MoE layer)
  for (long long e = (long long)blockIdx.x * kNumConsumers + c.tid; e < rows * nvec;
       e += (long long)gridDim.x * kNumConsumers) {
    const int tok = (int)(e / nvec), col = (int)(e % nvec) * 8;
    const size_t src = (size_t)tok * op.ld_in + (size_t)(col / bk) * 2 * bk + col % bk;
    float g[8], u[8], r[8];
    unpack8(__ldcg(reinterpret_cast<const uint4*>(in + src)), g);
    unpack8(__ldcg(reinterpret_cast<const uint4*>(in + src + bk)), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = rbf(g[i] / (1.0f + expf(-g[i]))) * u[i];
    *reinterpret_cast<uint4*>(out + (size_t)tok * op.ld_out + col) = pack8(r);
  }
}

__device__ ArgBest block_argmax(Ctx& c, ArgBest b) {
  float* scratch = c.red() + 32;
  b = warp_argmax(b);
  if (c.lane == 0) {
    scratch[c.warp * 2] = b.v;
    scratch[c.warp * 2 + 1] = __int_as_float(b.i);
  }
  consumer_sync();
  ArgBest a;
  a.v = scratch[0];
  a.i = __float_as_int(scratch[1]);
  for (int w = 1; w < kNumConsumerWarps; ++w) {
    ArgBest x;
    x.v = scratch[w * 2];
    x.i = __float_as_int(scratch[w * 2 + 1]);
    a = arg_better(a, x);
  }
  consumer_sync();
  return a;
}

// logits [T][n] -> amax_n partial (value, index) pairs per token
__device__ void op_argmax_partial(Ctx& c, const OpDesc& op, int T) {
  const int np = op.amax_n;
  const int chunk = (op.n + np - 1) / np;
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(op.in);
  for (int u = blockIdx.x; u < T * np; u += gridDim.x) {
    const int tok = u / np, ck = u % np;
    const int lo = ck * chunk, hi = min(op.n, lo + chunk);
    ArgBest b;
    b.v = -INFINITY;
    b.i = 0x7fffffff;
    for (int i = lo + c.tid; i < hi; i += kNumConsumers) {
      ArgBest x;
      x.v = __bfloat162float(__ldcg(in + (size_t)tok * op.ld_in + i));
      x.i = i;
      b = arg_better(b, x);
    }
    b = block_argmax(c, b);
    if (c.tid == 0) {
      op.amax_val[(size_t)tok * np + ck] = b.v;
      op.amax_idx[(size_t)tok * np + ck] = b.i;
    }
  }
}

// partial pairs -> int64 token per row; CTA 0 only
// Up to 8 tokens CTA 0 reduces them all: it also runs the bookkeeping that reads the result,
// so nothing has to cross CTAs.  Larger batches are spread over the grid (one token per CTA
// at a time) and pay one more grid barrier so that CTA 0 sees every token.
__device__ void op_argmax_reduce(Ctx& c, const OpDesc& op, int T) {
  long long* out = reinterpret_cast<long long*>(op.out);
  const bool spread = T > 8;
#if MK_WITH_XCHG
  const bool xrank = (op.flags & F_XRANK) != 0;  // aux0 = first vocabulary index of this rank's shard
#endif
  if (spread || blockIdx.x == 0) {
    for (int tok = spread ? blockIdx.x : 0; tok < T; tok += spread ? gridDim.x : 1) {
      ArgBest b;
      b.v = -INFINITY;
      b.i = 0x7fffffff;
      for (int i = c.tid; i < op.amax_n; i += kNumConsumers) {
        ArgBest x;
        x.v = __ldcg(op.amax_val + (size_t)tok * op.amax_n + i);
        x.i = __ldcg(op.amax_idx + (size_t)tok * op.amax_n + i);
        b = arg_better(b, x);
      }
      b = block_argmax(c, b);
#if MK_WITH_XCHG
      if (xrank && c.tid == 0) {
        // every rank tells every rank its best (value, global index) of the token; all pick the same winner
        // (larger value, then lower index: the shards are contiguous, so this is the unsharded rule)
        const KParams& p = c.p;
        const unsigned seq = xchg_next(c);
        if (b.i != 0x7fffffff) b.i += op.aux0;
        const size_t mine = (size_t)p.xchg_amax_word + ((size_t)p.rank * p.xchg_tokens + tok) * 2;
        for (int r = 0; r < p.world; ++r) {
          uint2* w = reinterpret_cast<uint2*>(p.xchg[r]) + mine;
          st_sys_v2(w, __float_as_uint(b.v), seq);
          st_sys_v2(w + 1, (uint32_t)b.i, seq);
        }
        ArgBest g;
        g.v = -INFINITY;
        g.i = 0x7fffffff;
        for (int r = 0; r < p.world; ++r) {
          const uint2* w = reinterpret_cast<const uint2*>(p.xchg[p.rank]) + (size_t)p.xchg_amax_word + ((size_t)r * p.xchg_tokens + tok) * 2;
          if (!xchg_wait_word(c, w, seq, r) || !xchg_wait_word(c, w + 1, seq, r)) break;
          ArgBest x;
          x.v = __uint_as_float(ld_sys_v2(w).x);
          x.i = (int)ld_sys_v2(w + 1).x;
          g = arg_better(g, x);
        }
        b = g;
      }
#endif
      if (c.tid == 0) out[(size_t)tok * op.ld_out] = (b.i == 0x7fffffff) ? -1 : (long long)b.i;
    }
  }
#if MK_WITH_XCHG
  if (xrank) c.ar_seq += 1;
#endif
  if (spread) grid_sync(c);
}


#if MK_WITH_MOE
// ------------------------------------------------------------------------------------
// mixture of experts (Qwen3-MoE decode, one or two batched tokens)
// ------------------------------------------------------------------------------------
// The reference runs routing, the two expert linears, SiLU*up and the weighted sum as tasks of their
// own (tasks/blackwell/topk_softmax_sm100.cuh, moe_linear_sm100.cuh, mul_sum_add_sm100.cuh).  Here, at
// one or two tokens, every (token, expert slot) pair is a GEMV: the expert linears run on the row-owner
// path over a VIRTUAL row space of pairs x rows-per-expert.  A CTA owns a contiguous range of it, walks
// it pair by pair in chunks of at most 32 rows, and the chunk's weight rows are the expert's rows of
// the [experts * rows, K] weight (the TMA row coordinate is expert * rows + row).  The producer can
// only run as far ahead as the routing is known: it waits for the consumers to pass the op's barrier.

// aux0 = top-k, aux1 = experts.  in: router logits [T, experts] bf16; amax_val / amax_idx: the runtime's
// routing tables [T, top-k] (fp32 weight, expert id).  One warp per token: fp32 softmax over the experts,
// k rounds of (largest probability, lowest index), weights renormalised over the k picked
// (transformers' Qwen3MoeTopKRouter with norm_topk_prob; reference task: topk_softmax_sm100.cuh:61-290).
// One token, by one warp: `w_out` / `idx_out` (may be null) receive the k weights and expert ids.
__device__ __noinline__ void moe_route_token(Ctx& c, const __nv_bfloat16* logits, int E, int K, float* w_out, int* idx_out, int* idx_out2) {
  float v[8];  // up to 256 experts: 8 per lane
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = c.lane + 32 * i;
    v[i] = e < E ? __bfloat162float(__ldcg(logits + e)) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = (c.lane + 32 * i) < E ? expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
  float picked_sum = 0.f, my_w = 0.f;
  int my_e = 0;
#pragma unroll 1
  for (int k = 0; k < K; ++k) {
    ArgBest b;
    b.v = -INFINITY;
    b.i = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ArgBest x;
      x.v = v[i] * inv;
      x.i = c.lane + 32 * i;
      if (x.i < E && v[i] >= 0.f) b = arg_better(b, x);
    }
    b = warp_argmax(b);
    picked_sum += b.v;
    if (c.lane == k) {
      my_w = b.v;
      my_e = b.i;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c.lane + 32 * i == b.i) v[i] = -1.f;  // taken
  }
  if (c.lane < K) {
    if (w_out != nullptr) w_out[c.lane] = my_w / picked_sum;
    if (idx_out != nullptr) idx_out[c.lane] = my_e;
    if (idx_out2 != nullptr) idx_out2[c.lane] = my_e;
  }
}
__device__ __noinline__ void op_moe_route(Ctx& c, const OpDesc& op, int T) {
  const int E = op.aux1, K = op.aux0;
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(op.in);
#pragma unroll 1
  for (int t = blockIdx.x * kNumConsumerWarps + c.warp; t < T; t += gridDim.x * kNumConsumerWarps)
    moe_route_token(c, in + (size_t)t * op.ld_in, E, K, op.amax_val + (size_t)t * K, op.amax_idx + (size_t)t * K, nullptr);
}

// The CTA's share of the virtual row space of a MoE linear and its walk: pairs x n rows, contiguous ranges
// of 8-row units per CTA, segments that end at pair boundaries, chunks of at most 32 rows inside a segment.
struct MoeWalk {
  int row0, row1;  // the CTA's virtual rows
  int n;           // rows per expert (= per pair)
  bool any;
};
__device__ __forceinline__ MoeWalk moe_walk(const OpDesc& op, int pairs) {
  MoeWalk w;
  w.n = op.n;
  const unsigned U = (unsigned)pairs * (unsigned)(op.n / kUnitRows);
  const unsigned G = min((unsigned)gridDim.x, U);
  w.any = blockIdx.x < G;
  w.row0 = w.any ? (int)tile_begin(blockIdx.x, U, G) * kUnitRows : 0;
  w.row1 = w.any ? (int)tile_begin(blockIdx.x + 1, U, G) * kUnitRows : 0;
  return w;
}

__device__ __noinline__ void op_moe_down_combine(Ctx& c, const OpDesc& op, int T);

// aux0 = top-k, aux1 = experts, n = rows per expert, k = K.  w: [experts * n, K] bf16 (tmap_w: the four maps of
// the row-owner path over that 2-D view).  in: [T, K] (one row per token) or, with F_MOE_PAIR_IN, [T * top-k, K];
// out: [T * top-k, n].  amax_idx: the routing table.
__device__ __noinline__ void op_moe_linear(Ctx& c, const OpDesc& op, int T) {
  const KParams& p = c.p;
  if (op_barrier(c, op)) return;
  const int topk = op.aux0;
  if (op.flags & F_MOE_ROUTE) {
    // The routing folded into this op: warp t of EVERY CTA routes token t from the router logits (one or two
    // tokens) and leaves the expert ids in shared memory for this CTA's producer; CTA 0 also stores the
    // runtime's tables, which the later ops of the layer read behind their barriers.
    int* rt = reinterpret_cast<int*>(c.smem + p.x_off + p.x_bytes - 512);
    if (c.warp < T)
      moe_route_token(c, reinterpret_cast<const __nv_bfloat16*>(op.res) + (size_t)c.warp * op.ld_res, op.aux1, topk,
                      blockIdx.x == 0 ? op.amax_val + (size_t)c.warp * topk : nullptr,
                      blockIdx.x == 0 ? op.amax_idx + (size_t)c.warp * topk : nullptr, rt + c.warp * topk);
    consumer_sync();
    __threadfence_block();
  }
  c.lin_seq += 1;
  if (c.tid == 0) c.flags()[4] = (int)c.lin_seq;  // the routing is visible: the producer may pick this op's expert rows
  if (op.flags & F_MOE_COMBINE) {
    op_moe_down_combine(c, op, T);
    return;
  }
  const int pairs = T * topk;
  const MoeWalk wk = moe_walk(op, pairs);
  if (!wk.any || wk.row0 >= wk.row1) return;
  const int nks = op.nkt;
  const int kp = nks * kRowsStageK;
  const bool pair_in = (op.flags & F_MOE_PAIR_IN) != 0;
  const int p_first = wk.row0 / wk.n, p_last = (wk.row1 - 1) / wk.n;
  // input rows this CTA needs: those of its pairs (the down projection) or of their tokens
  const int in_first = pair_in ? p_first : p_first / topk;
  const int in_last = pair_in ? p_last : p_last / topk;
  const int nrows = in_last - in_first + 1;  // at most 8 (the host admits MoE graphs for one or two tokens)
  stage_x(c, reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)in_first * op.ld_in, op.ld_in, op.k, kp,
          (op.flags & F_NORM_IN) ? op.norm_w : nullptr, 0, nrows, nrows, nullptr);
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  const int pitch_b = (kp + 8) * 2;
  const uint32_t xs0 = c.smem_addr + p.x_off;
  const uint32_t x_zero = xs0 + (uint32_t)(nrows * pitch_b);
  const uint32_t w_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
  const uint32_t w_xor = (uint32_t)(lane & 7);
  const uint32_t w_hi = (uint32_t)(lane >> 4);
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0);
  const int TP = p.sums_stride;
  float* sums = c.sums();
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  const int e_row = c.tid & 31;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
#pragma unroll 1
  for (int pr = p_first; pr <= p_last; ++pr) {
    const int seg0 = max(wk.row0, pr * wk.n), seg1 = min(wk.row1, (pr + 1) * wk.n);
    const int nch = rows_num_chunks(seg0, seg1);
    // the B operand of the mma: column 0 = the pair's input row, the other seven columns zero
    const int xrow = (pair_in ? pr : pr / topk) - in_first;
    const bool a_real = (lane & 7) == 0;
    const uint32_t a_row = a_real ? xs0 + (uint32_t)(xrow * pitch_b + (lane >> 3) * 16 + warp * 128) : x_zero;
#pragma unroll 1
    for (int ci = 0; ci < nch; ++ci) {
      const int r0 = rows_chunk_begin(seg0, seg1, nch, ci);
      const int R = rows_chunk_begin(seg0, seg1, nch, ci + 1) - r0;
      const int ntile = (R + 15) >> 4;
      float acc[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
      const uint32_t box_bytes = (uint32_t)R * 128u;
#pragma unroll 1
      for (int ks = 0; ks < nks; ++ks) {
        mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
        const uint32_t wb = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes + (uint32_t)warp * box_bytes + w_off;
        const uint32_t xa = a_row + (a_real ? (uint32_t)(ks * kRowsStageK * 2) : 0u);
        uint32_t x[2][4];
        ldmatrix_x4(xa, x[0][0], x[0][1], x[0][2], x[0][3]);
        ldmatrix_x4(xa + (a_real ? 64u : 0u), x[1][0], x[1][1], x[1][2], x[1][3]);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (t < ntile) {
#pragma unroll
            for (int st = 0; st < 4; ++st) {
              uint32_t w0, w1, w2, w3;
              ldmatrix_x4(wb + (uint32_t)t * 2048u + ((((uint32_t)(2 * st) + w_hi) ^ w_xor) << 4), w0, w1, w2, w3);
              mma_bf16(acc[2 * t + (st & 1)], w0, w1, w2, w3, x[st >> 1][2 * (st & 1)], x[st >> 1][2 * (st & 1) + 1]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty0 + 8 * s);
        ++consumed;
        if (++s == S) {
          s = 0;
          parity ^= 1u;
        }
      }
      // column 0 of the accumulators (lanes with (lane & 3) == 0): rows 16t + (lane >> 2) and + 8
      if ((lane & 3) == 0) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          float* d = sums + ((warp * kChunkRows + 16 * t + (lane >> 2)) * TP);
          d[0] = acc[2 * t][0] + acc[2 * t + 1][0];
          d[8 * TP] = acc[2 * t][2] + acc[2 * t + 1][2];
        }
      }
      consumer_sync();
      if (c.tid < 32 && e_row < R) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kNumConsumerWarps; ++w) v += sums[(w * kChunkRows + e_row) * TP];
        out[(size_t)pr * op.ld_out + (r0 - pr * wk.n) + e_row] = __float2bfloat16_rn(v);
      }
      consumer_sync();
    }
  }
  c.cons_idx += consumed;
}

// The down projection of the experts with the weighted sum folded in (F_MOE_COMBINE).  A CTA owns a range of the n
// OUTPUT rows for all expert slots of a token: per token it stages the token's top-k input rows, then per chunk of
// rows walks the slots (the weight rows are the slot's expert's rows of that chunk), rounds each slot's sums to bf16
// like the linear's output would be, and adds them up slot by slot exactly as the stand-alone weighted sum does
// (bf16 roundings of the PyTorch model, or fp32 fused multiply-adds), + residual.  The per-slot sums of the warps
// alternate between the two token slots of the sums block, so that one CTA-wide sync per slot is enough.
__device__ __noinline__ void op_moe_down_combine(Ctx& c, const OpDesc& op, int T) {
  const KParams& p = c.p;
  const int topk = op.aux0;
  int row0, row1;
  bool any;
  rows_range(op, row0, row1, any);
  if (!any || row0 >= row1) return;
  const int nks = op.nkt;
  const int kp = nks * kRowsStageK;
  const int S = p.num_stages;
  const int lane = c.lane, warp = c.warp;
  const int pitch_b = (kp + 8) * 2;
  const uint32_t xs0 = c.smem_addr + p.x_off;
  const uint32_t x_zero = xs0 + (uint32_t)(topk * pitch_b);
  const uint32_t w_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * 128);
  const uint32_t w_xor = (uint32_t)(lane & 7);
  const uint32_t w_hi = (uint32_t)(lane >> 4);
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0);
  const int TP = p.sums_stride;  // 2
  float* sums = c.sums();
  const bool torch_num = p.numerics == NUM_TORCH;
  const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(op.res);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  const int e_row = c.tid & 31;
  int s = (int)(c.cons_idx % (unsigned)S);
  uint32_t parity = (c.cons_idx / (unsigned)S) & 1u;
  unsigned consumed = 0;
  const int nch = rows_num_chunks(row0, row1);
#pragma unroll 1
  for (int t = 0; t < T; ++t) {
    stage_x(c, reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)t * topk * op.ld_in, op.ld_in, op.k, kp, nullptr, 0, topk, topk, nullptr);
#pragma unroll 1
    for (int ci = 0; ci < nch; ++ci) {
      const int r0 = rows_chunk_begin(row0, row1, nch, ci);
      const int R = rows_chunk_begin(row0, row1, nch, ci + 1) - r0;
      const int ntile = (R + 15) >> 4;
      const uint32_t box_bytes = (uint32_t)R * 128u;
      float comb = 0.f;  // (threads 0..R-1: the running weighted sum of output row r0 + tid)
      float rr = 0.f;
      if (c.tid < R && res != nullptr) rr = __bfloat162float(__ldcg(res + (size_t)t * op.ld_res + r0 + e_row));
#pragma unroll 1
      for (int sl = 0; sl < topk; ++sl) {
        const bool a_real = (lane & 7) == 0;
        const uint32_t a_row = a_real ? xs0 + (uint32_t)(sl * pitch_b + (lane >> 3) * 16 + warp * 128) : x_zero;
        float acc[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
#pragma unroll 1
        for (int ks = 0; ks < nks; ++ks) {
          mbar_wait(c, bar_full0 + 8 * s, parity, ST_TIMEOUT_FULL);
          const uint32_t wb = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes + (uint32_t)warp * box_bytes + w_off;
          const uint32_t xa = a_row + (a_real ? (uint32_t)(ks * kRowsStageK * 2) : 0u);
          uint32_t x[2][4];
          ldmatrix_x4(xa, x[0][0], x[0][1], x[0][2], x[0][3]);
          ldmatrix_x4(xa + (a_real ? 64u : 0u), x[1][0], x[1][1], x[1][2], x[1][3]);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (q < ntile) {
#pragma unroll
              for (int st = 0; st < 4; ++st) {
                uint32_t w0, w1, w2, w3;
                ldmatrix_x4(wb + (uint32_t)q * 2048u + ((((uint32_t)(2 * st) + w_hi) ^ w_xor) << 4), w0, w1, w2, w3);
                mma_bf16(acc[2 * q + (st & 1)], w0, w1, w2, w3, x[st >> 1][2 * (st & 1)], x[st >> 1][2 * (st & 1) + 1]);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty0 + 8 * s);
          ++consumed;
          if (++s == S) {
            s = 0;
            parity ^= 1u;
          }
        }
        const int half = sl & 1;
        if ((lane & 3) == 0) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float* d = sums + ((warp * kChunkRows + 16 * q + (lane >> 2)) * TP) + half;
            d[0] = acc[2 * q][0] + acc[2 * q + 1][0];
            d[8 * TP] = acc[2 * q][2] + acc[2 * q + 1][2];
          }
        }
        consumer_sync();
        if (c.tid < R) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kNumConsumerWarps; ++w) v += sums[(w * kChunkRows + e_row) * TP + half];
          const float f = rbf(v);  // the down projection's output is bf16
          const float wgt = __ldcg(op.amax_val + (size_t)t * topk + sl);
          comb = torch_num ? rbf(comb + rbf(f * wgt)) : fmaf(f, wgt, comb);
        }
      }
      if (c.tid < R) {
        float v = comb;
        if (res != nullptr) v = (torch_num ? rbf(v) : v) + rr;
        out[(size_t)t * op.ld_out + r0 + e_row] = __float2bfloat16_rn(v);
      }
      consumer_sync();  // (the next chunk's or token's first slot writes the half the last slot may still be read from)
    }
  }
  c.cons_idx += consumed;
}

// aux0 = top-k.  in: [T * top-k, n] bf16, amax_val: routing weights [T, top-k], res: [T, n] (may be null), out: [T, n].
// out[t] = bf16( sum over the token's slots of weight * in[pair] ) + residual  (reference task mul_sum_add_sm100.cuh:17-48;
// the PyTorch model adds the slots up in bf16 and the residual in bf16)
__device__ void op_moe_combine(Ctx& c, const OpDesc& op, int T) {
  const int topk = op.aux0;
  const int nvec = op.n >> 3;
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(op.in);
  const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(op.res);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(op.out);
  const bool torch_num = c.p.numerics == NUM_TORCH;
#pragma unroll 1
  for (int u = blockIdx.x * kNumConsumers + c.tid; u < T * nvec; u += gridDim.x * kNumConsumers) {
    const int t = u / nvec, v = u % nvec;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 1
    for (int sl = 0; sl < topk; ++sl) {
      const float wgt = __ldcg(op.amax_val + (size_t)t * topk + sl);
      float f[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(in + (size_t)(t * topk + sl) * op.ld_in) + v), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = torch_num ? rbf(acc[i] + rbf(f[i] * wgt)) : fmaf(f[i], wgt, acc[i]);
    }
    if (res != nullptr) {
      float r[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(res + (size_t)t * op.ld_res) + v), r);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = (torch_num ? rbf(acc[i]) : acc[i]) + r[i];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * op.ld_out)[v] = pack8(acc);
  }
}
#endif  // MK_WITH_MOE

// ------------------------------------------------------------------------------------
// stand-alone allreduce layer
// ------------------------------------------------------------------------------------
// aux0 = world size, aux1 = this rank.  in: this rank's partial sums [T, n] bf16, out: the sum over
// ranks [T, n] bf16 (fp32 addition in rank order, one rounding: the reference's reduction task,
// tasks/ampere/reduction.cuh:139-166).  The host lowers an allreduce layer to this op only where it
// cannot fold the exchange into the producing linear's epilogue and the consumers' input staging
// (F_PUSH / F_GATHER_*).  Same exchange words as there: every unit of 8 columns is pushed to all
// ranks and then gathered from this rank's own region by the same thread.
__device__ __noinline__ void op_allreduce(Ctx& c, const OpDesc& op, int T) {
  const KParams& p = c.p;
  if (op_barrier(c, op)) return;
  const int world = op.aux0;
  const int nvec = op.n >> 3;
  if (world <= 1) {  // a single rank: the sum is the input
#pragma unroll 1
    for (int u = blockIdx.x * kNumConsumers + c.tid; u < T * nvec; u += gridDim.x * kNumConsumers) {
      const int row = u / nvec, v = u % nvec;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)row * op.ld_out)[v] =
          __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)row * op.ld_in) + v);
    }
    return;
  }
#if MK_WITH_XCHG
  const unsigned seq = xchg_next(c);
#pragma unroll 1
  for (int u = blockIdx.x * kNumConsumers + c.tid; u < T * nvec; u += gridDim.x * kNumConsumers) {
    const int row = u / nvec, v = u % nvec;
    float f[8];
    unpack8(__ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.in) + (size_t)row * op.ld_in) + v), f);
    const size_t w = xchg_word(seq, p.world, p.xchg_tokens, p.xchg_cols, p.rank, row, v * 8);
#pragma unroll 1
    for (int r = 0; r < world; ++r) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(p.xchg[r]) + w);
#pragma unroll
      for (int i = 0; i < 4; ++i) st_sys_v4(dst + i, __float_as_uint(f[2 * i]), seq, __float_as_uint(f[2 * i + 1]), seq);
    }
    reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(op.out) + (size_t)row * op.ld_out)[v] = xchg_gather8(c, seq, row, v * 8);
  }
  c.ar_seq += 1;
#endif  // (the host launches the tensor-parallel build of this kernel whenever world > 1)
}

// ------------------------------------------------------------------------------------
// continuous-batching bookkeeping between iterations (CTA 0, one thread)
// ------------------------------------------------------------------------------------
// Same protocol as the reference's offline mode (persistent_kernel.cuh:380-536):
// append the sampled tokens, retire finished requests and free their pages,
// compact the survivors, give each one more token, admit new requests, and
// leave the number of active tokens in qo_indptr[max_reqs].  It is split in two so
// that a launch bounded by max_iters still appends its last tokens before it ends.
// Part 1, after an iteration: append the sampled tokens, advance step[], retire
// finished requests and return their pages.
__device__ __noinline__ void bookkeep_finish(Ctx& c) {
  const KParams& p = c.p;
  const int R = p.max_reqs;
  int tail = p.sched[1];
  for (int i = 0; i < R; ++i) {
    const int rid = p.request_ids[i];
    if (rid < 0) continue;
    int st = p.step[rid];
    const int q0 = p.qo_indptr[i];
    const int n = p.qo_indptr[i + 1] - q0;
    const int pl = p.prompt_lengths[rid];
    for (int j = 0; j < n; ++j) {
      const int pos = st + j + 1;
      if (pos >= pl && pos < p.max_seq_len) p.tokens[(size_t)rid * p.max_seq_len + pos] = p.output_tokens[q0 + j];
    }
    st += n;
    p.step[rid] = st;
    const bool done = (st + 1 >= p.max_seq_len) ||
                      (st >= pl && p.tokens[(size_t)rid * p.max_seq_len + st] == p.eos);
    if (done) {
      p.request_ids[i] = -1;
      const int k0 = p.kv_indptr[i], k1 = p.kv_indptr[i + 1];
      for (int j = k0; j < k1; ++j) {
        p.page_queue[tail % p.max_pages] = p.kv_indices[j];
        ++tail;
      }
    }
  }
  p.sched[1] = tail;
}

// Part 2, before an iteration: compact the surviving requests, give each one more
// token and the page it needs, admit new requests.  Returns the active tokens.
__device__ __noinline__ int bookkeep_prepare(Ctx& c) {
  const KParams& p = c.p;
  const int R = p.max_reqs;
  int head = p.sched[0], tail = p.sched[1];
  int* old_idx = reinterpret_cast<int*>(c.smem + p.x_off);
  const int n_old = p.kv_indptr[R];
  for (int i = 0; i < n_old; ++i) old_idx[i] = p.kv_indices[i];
  int nreq = 0, ntok = 0, npages = 0;
  for (int i = 0; i < R; ++i) {
    const int rid = p.request_ids[i];
    if (rid < 0) continue;
    const int k0 = p.kv_indptr[i];
    const int have = p.kv_indptr[i + 1] - k0;
    p.request_ids[nreq] = rid;
    p.qo_indptr[nreq] = ntok;
    p.kv_indptr[nreq] = npages;
    const int st = p.step[rid];
    // a request still inside its prompt gets a chunk of it (as many tokens as the budget allows), a
    // decoding one its single token; either may get nothing when the iteration's budget is spent
    const int left = p.prompt_lengths[rid] - st;
    const int budget = p.max_tokens - ntok;
    const int nnew = left > 0 ? min(left, min(p.max_tokens_per_req, budget)) : min(1, budget);
    for (int j = 0; j < nnew; ++j) p.input_tokens[ntok + j] = p.tokens[(size_t)rid * p.max_seq_len + st + j];
    const int need = (st + nnew + p.page_size - 1) / p.page_size;
    const int last = (st + nnew) % p.page_size;
    p.kv_last_page_len[nreq] = last == 0 ? p.page_size : last;
    for (int j = 0; j < have; ++j) p.kv_indices[npages + j] = old_idx[k0 + j];
    for (int j = have; j < need; ++j) {
      if (tail - head <= 0) {
        raise_abort(c, ST_OUT_OF_PAGES, rid, need);
        return 0;
      }
      p.kv_indices[npages + j] = p.page_queue[head % p.max_pages];
      ++head;
    }
    npages += need > have ? need : have;
    ntok += nnew;
    ++nreq;
  }
  while (nreq < R && ntok < p.max_tokens) {
    const int rid = p.sched[2];
    if (rid >= p.total_requests) break;
    const int nnew = max(1, min(p.prompt_lengths[rid], min(p.max_tokens_per_req, p.max_tokens - ntok)));
    const int need = (nnew + p.page_size - 1) / p.page_size;
    if (tail - head < need) break;  // no pages for a new request yet: admit it later
    p.request_ids[nreq] = rid;
    p.qo_indptr[nreq] = ntok;
    p.kv_indptr[nreq] = npages;
    for (int j = 0; j < nnew; ++j) p.input_tokens[ntok + j] = p.tokens[(size_t)rid * p.max_seq_len + j];
    const int last = nnew % p.page_size;
    p.kv_last_page_len[nreq] = last == 0 ? p.page_size : last;
    for (int j = 0; j < need; ++j) {
      p.kv_indices[npages + j] = p.page_queue[head % p.max_pages];
      ++head;
    }
    npages += need;
    ntok += nnew;
    ++nreq;
    p.sched[2] = rid + 1;
  }
  for (int i = nreq; i < R; ++i) p.request_ids[i] = -1;
  for (int i = nreq; i <= R; ++i) {
    p.qo_indptr[i] = ntok;
    p.kv_indptr[i] = npages;
  }
  p.sched[0] = head;
  p.sched[1] = tail;
  return ntok;
}

// ------------------------------------------------------------------------------------
// the TMA producer
// ------------------------------------------------------------------------------------
// Position in this CTA's weight-tile sequence: the linear ops in program order, each
// with the CTA's contiguous tile range.
struct TileCursor {
  int oi;
  unsigned tile, t1;
  int blk, kt, nkt;
  const void* tmap;
  bool valid;
};

// Open the CTA's range of linear op `oi`; false if the op is not linear or gives this CTA nothing.
__device__ __forceinline__ bool cursor_open(const KParams& p, TileCursor& tc, int oi) {
  const OpDesc& op = p.ops[oi];
  if (op.type != OP_LINEAR || (op.flags & F_ROWS)) return false;
  const unsigned total = (unsigned)op.nblk * (unsigned)op.nkt;
  const int G = (int)min(gridDim.x, total);
  if ((int)blockIdx.x >= G) return false;
  tc.oi = oi;
  tc.tile = tile_begin(blockIdx.x, total, G);
  tc.t1 = tile_begin(blockIdx.x + 1, total, G);
  tc.nkt = op.nkt;
  tc.blk = (int)(tc.tile / (unsigned)op.nkt);
  tc.kt = (int)(tc.tile - (unsigned)tc.blk * (unsigned)op.nkt);
  tc.tmap = op.tmap_w;
  return tc.tile < tc.t1;
}

// Step the look-ahead cursor one tile, wrapping from the last linear op to the first
// (the next iteration streams the same weights).
__device__ __forceinline__ void cursor_advance_wrap(const KParams& p, TileCursor& tc) {
  tc.tile += 1;
  if (++tc.kt == tc.nkt) {
    tc.kt = 0;
    tc.blk += 1;
  }
  if (tc.tile < tc.t1) return;
  int oi = tc.oi;
  for (int n = 0; n < p.num_ops; ++n) {
    oi = (oi + 1 == p.num_ops) ? 0 : oi + 1;
    if (cursor_open(p, tc, oi)) return;
  }
  tc.valid = false;
}

// Position in this CTA's sequence of row-owner stages (op, chunk, k stage), used by the L2
// look-ahead of the producer; wraps from the last linear op to the first.
struct RowsCursor {
  int oi, row0, row1, nch, ci, ks, nks;
  bool valid;
};
__device__ __forceinline__ bool rows_cursor_open(const KParams& p, RowsCursor& rc, int oi) {
  const OpDesc& op = p.ops[oi];
  if (op.type != OP_LINEAR || !(op.flags & F_ROWS)) return false;
  int row0, row1;
  bool any;
  rows_range(op, row0, row1, any);
  if (!any || row0 >= row1) return false;
  rc.oi = oi;
  rc.row0 = row0;
  rc.row1 = row1;
  rc.nch = rows_num_chunks(row0, row1);
  rc.ci = 0;
  rc.ks = 0;
  rc.nks = op.nkt;
  return true;
}
__device__ __forceinline__ void rows_cursor_next(const KParams& p, RowsCursor& rc) {
  if (++rc.ks < rc.nks) return;
  rc.ks = 0;
  if (++rc.ci < rc.nch) return;
  int oi = rc.oi;
  for (int n = 0; n < p.num_ops; ++n) {
    oi = (oi + 1 == p.num_ops) ? 0 : oi + 1;
    if (rows_cursor_open(p, rc, oi)) return;
  }
  rc.valid = false;
}
// L2 look-ahead of the row-owner weight stream, run by the 32 lanes of the (otherwise idle)
// activation-producer warp: the stages the ring will load next are requested into L2 line by
// line with plain prefetch instructions, so that HBM keeps streaming while the consumers sit
// in a barrier or stage their inputs, and the ring refills from L2 when they come back.
__device__ __noinline__ void rows_prefetch_loop(Ctx& c) {
  const KParams& p = c.p;
  if (p.prefetch_tiles <= 0) return;
  const unsigned W = (unsigned)p.prefetch_tiles;
  volatile int* fl = c.flags();
  RowsCursor rc;
  rc.valid = false;
  for (int oi = 0; oi < p.num_ops && !rc.valid; ++oi) rc.valid = rows_cursor_open(p, rc, oi);
  unsigned pos = 0;  // the cursor's index in this CTA's stage sequence
  while (rc.valid) {
    if (fl[0] < 0) break;  // the consumers have left
    const unsigned issued = (unsigned)fl[1];
    if (pos >= issued + W) {
      __nanosleep(200);
      continue;
    }
    if (pos >= issued) {
      const OpDesc& op = p.ops[rc.oi];
      const int r0 = rows_chunk_begin(rc.row0, rc.row1, rc.nch, rc.ci);
      const int R = rows_chunk_begin(rc.row0, rc.row1, rc.nch, rc.ci + 1) - r0;
      const unsigned char* w = reinterpret_cast<const unsigned char*>(op.w);
      for (int idx = c.lane; idx < R * 8; idx += 32) {
        const int row = r0 + (idx >> 3), kk = rc.ks * kRowsStageK + (idx & 7) * 64;
        if (row < op.n && kk < op.k) {
          const unsigned char* a = w + ((size_t)row * op.ld_out2 + kk) * 2;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
        }
      }
    }
    rows_cursor_next(p, rc);
    ++pos;
  }
}

template <int PATH>
__device__ __noinline__ void producer_loop(Ctx& c) {
  const KParams& p = c.p;
  const int S = p.num_stages;
  volatile int* fl = c.flags();
  unsigned issued = 0;
  int s = 0;
  uint32_t empty_parity = 1;  // a fresh barrier passes a wait on the "previous" phase
#if MK_WITH_MOE
  unsigned lin_seq = 0;       // linear and MoE-linear ops seen so far in this launch (the consumers count the same way)
#endif
  const uint32_t bar_full0 = c.full_bar(0), bar_empty0 = c.empty_bar(0);
  // look-ahead: tiles beyond the shared-memory ring are requested into L2 so that HBM
  // keeps streaming while the consumers sit in barriers, staging and epilogues
  TileCursor pc;
  pc.valid = false;
  int ahead = 0;
  if (PATH != PATH_ROWS && p.prefetch_tiles > 0)
    for (int oi = 0; oi < p.num_ops && !pc.valid; ++oi) pc.valid = cursor_open(p, pc, oi);
  // Weights are read once per step: their lines are marked evict-first on the way through L2, so
  // that what the look-ahead has fetched (and the KV cache) is not pushed out by bytes already used.
  uint64_t pol_stream;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_stream));
  for (int iter = 1;; ++iter) {
    // wait for the consumers to publish this iteration's token count (or the end)
    int go;
    {
      unsigned long long t0 = 0;
      int spins = 0;
      while (true) {
        go = fl[0];
        if (go < 0 || (go >> 8) >= iter) break;
        __nanosleep(40);
        if (((++spins) & 255) == 0) {
          if (aborted(c)) { go = -1; break; }
          const unsigned long long now = globaltimer();
          if (t0 == 0) t0 = now;
          if (now - t0 > 4 * c.p.timeout_ns) {
            raise_abort(c, ST_TIMEOUT_GO, iter, go);
            go = -1;
            break;
          }
        }
      }
    }
    if (go < 0) break;
    const int T = go & 255;
    bool dead = false;
    for (int oi = 0; oi < p.num_ops && !dead; ++oi) {
      const OpDesc& rop = p.ops[oi];
      if constexpr (PATH == PATH_ROWS) {
#if MK_WITH_MOE
        if (rop.type == OP_MOE_LINEAR) {
          // the expert of a pair is only known once the consumers have passed this op's barrier
          lin_seq += 1;
          {
            unsigned long long t0 = 0;
            int spins = 0;
            while ((unsigned)fl[4] < lin_seq) {
              if (fl[0] < 0) { dead = true; break; }
              __nanosleep(40);
              if (((++spins) & 1023) == 0) {
                if (aborted(c)) { dead = true; break; }
                const unsigned long long now = globaltimer();
                if (t0 == 0) t0 = now;
                if (now - t0 > 4 * c.p.timeout_ns) { dead = true; break; }
              }
            }
          }
          if (dead) break;
          __threadfence();
          const int topk = rop.aux0;
          if (rop.flags & F_MOE_COMBINE) {
            // output rows owned for all slots: token, chunk of rows, slot, k stage (the consumers' order)
            int row0, row1;
            bool any;
            rows_range(rop, row0, row1, any);
            if (!any || row0 >= row1) continue;
            const int nch = rows_num_chunks(row0, row1);
            for (int t = 0; t < T && !dead; ++t)
              for (int ci = 0; ci < nch && !dead; ++ci) {
                const int r0 = rows_chunk_begin(row0, row1, nch, ci);
                const int R = rows_chunk_begin(row0, row1, nch, ci + 1) - r0;
                const void* tmap = reinterpret_cast<const unsigned char*>(rop.tmap_w) + ((R >> 3) - 1) * 128;
                const uint32_t box_bytes = (uint32_t)R * 128u;
                for (int sl = 0; sl < topk && !dead; ++sl) {
                  const int wrow = __ldcg(rop.amax_idx + t * topk + sl) * rop.n + r0;
                  for (int ks = 0; ks < rop.nkt; ++ks) {
                    if (!mbar_wait(c, bar_empty0 + 8 * s, empty_parity, ST_TIMEOUT_EMPTY)) {
                      dead = true;
                      break;
                    }
                    const uint32_t full = bar_full0 + 8 * s;
                    const uint32_t dst = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
                    mbar_arrive_expect_tx(full, 8u * box_bytes);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                      tma_load_2d_hint(dst + (uint32_t)j * box_bytes, tmap, full, ks * kRowsStageK + j * kBoxK, wrow, pol_stream);
                    issued += 1;
                    fl[1] = (int)issued;
                    if (++s == S) {
                      s = 0;
                      empty_parity ^= 1u;
                    }
                  }
                }
              }
            continue;
          }
          const MoeWalk wk = moe_walk(rop, T * topk);
          if (!wk.any || wk.row0 >= wk.row1) continue;
          const int p_first = wk.row0 / wk.n, p_last = (wk.row1 - 1) / wk.n;
          for (int pr = p_first; pr <= p_last && !dead; ++pr) {
            const int expert = (rop.flags & F_MOE_ROUTE) ? reinterpret_cast<volatile int*>(c.smem + p.x_off + p.x_bytes - 512)[pr]
                                                         : __ldcg(rop.amax_idx + pr);
            const int seg0 = max(wk.row0, pr * wk.n), seg1 = min(wk.row1, (pr + 1) * wk.n);
            const int nch = rows_num_chunks(seg0, seg1);
            for (int ci = 0; ci < nch && !dead; ++ci) {
              const int r0 = rows_chunk_begin(seg0, seg1, nch, ci);
              const int R = rows_chunk_begin(seg0, seg1, nch, ci + 1) - r0;
              const void* tmap = reinterpret_cast<const unsigned char*>(rop.tmap_w) + ((R >> 3) - 1) * 128;
              const uint32_t box_bytes = (uint32_t)R * 128u;
              const int wrow = expert * wk.n + (r0 - pr * wk.n);  // the chunk's first row in the [experts * n, K] weight
              for (int ks = 0; ks < rop.nkt; ++ks) {
                if (!mbar_wait(c, bar_empty0 + 8 * s, empty_parity, ST_TIMEOUT_EMPTY)) {
                  dead = true;
                  break;
                }
                const uint32_t full = bar_full0 + 8 * s;
                const uint32_t dst = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
                mbar_arrive_expect_tx(full, 8u * box_bytes);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  tma_load_2d_hint(dst + (uint32_t)j * box_bytes, tmap, full, ks * kRowsStageK + j * kBoxK, wrow, pol_stream);
                issued += 1;
                fl[1] = (int)issued;
                if (++s == S) {
                  s = 0;
                  empty_parity ^= 1u;
                }
              }
            }
          }
          continue;
        }
        if (rop.type == OP_LINEAR) lin_seq += 1;
#endif
        if (rop.type != OP_LINEAR) continue;
        // row-owner op: per chunk of up to 32 owned rows, the full K in 512-wide stages of
        // eight boxes; the tensor map for a chunk of R rows is the (R / 8)-th of the op's four
        int row0, row1;
        bool any;
        rows_range(rop, row0, row1, any);
        if (!any) continue;
        const int passes = linear_passes(rop, T);
        const int nch = rows_num_chunks(row0, row1);
        for (int g = 0; g < passes && !dead; ++g)
          for (int ci = 0; ci < nch && !dead; ++ci) {
            const int r0 = rows_chunk_begin(row0, row1, nch, ci);
            const int R = rows_chunk_begin(row0, row1, nch, ci + 1) - r0;
            const void* tmap = reinterpret_cast<const unsigned char*>(rop.tmap_w) + ((R >> 3) - 1) * 128;
            const uint32_t box_bytes = (uint32_t)R * 128u;
            for (int ks = 0; ks < rop.nkt; ++ks) {
              if (!mbar_wait(c, bar_empty0 + 8 * s, empty_parity, ST_TIMEOUT_EMPTY)) {
                dead = true;
                break;
              }
              const uint32_t full = bar_full0 + 8 * s;
              const uint32_t dst = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
              mbar_arrive_expect_tx(full, 8u * box_bytes);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                tma_load_2d_hint(dst + (uint32_t)j * box_bytes, tmap, full, ks * kRowsStageK + j * kBoxK, r0, pol_stream);
              issued += 1;
              fl[1] = (int)issued;
              if (++s == S) {
                s = 0;
                empty_parity ^= 1u;
              }
            }
          }
        continue;
      } else {
      TileCursor lc;
      if (!cursor_open(p, lc, oi)) continue;
      const int passes = linear_passes(p.ops[oi], T);
      const unsigned t0 = lc.tile;
      for (int g = 0; g < passes && !dead; ++g) {
        if (g > 0) cursor_open(p, lc, oi);
        for (unsigned tile = t0; tile < lc.t1; ++tile) {
          if (g == 0 && pc.valid) {
            while (ahead < p.prefetch_tiles) {
              tma_prefetch_2d(pc.tmap, pc.kt * kTileK, pc.blk * kTileRows);
              tma_prefetch_2d(pc.tmap, pc.kt * kTileK + kBoxK, pc.blk * kTileRows);
              cursor_advance_wrap(p, pc);
              ++ahead;
            }
            --ahead;
          }
          if (!mbar_wait(c, bar_empty0 + 8 * s, empty_parity, ST_TIMEOUT_EMPTY)) {
            dead = true;
            break;
          }
          const uint32_t full = bar_full0 + 8 * s;
          const uint32_t dst = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
          mbar_arrive_expect_tx(full, kStageBytes);
          tma_load_2d_hint(dst, lc.tmap, full, lc.kt * kTileK, lc.blk * kTileRows, pol_stream);
          tma_load_2d_hint(dst + kSubBytes, lc.tmap, full, lc.kt * kTileK + kBoxK, lc.blk * kTileRows, pol_stream);
          issued += 1;
          fl[1] = (int)issued;
          if (++s == S) {
            s = 0;
            empty_parity ^= 1u;
          }
          if (++lc.kt == lc.nkt) {
            lc.kt = 0;
            lc.blk += 1;
          }
        }
      }
      }  // stream-K paths
    }
    if (dead || p.mode == MODE_ONEPASS) break;
  }
  fl[1] = (int)issued;
}

// The activation producer (warp 9, one lane).  For wide-batch linear ops it walks the same
// tile sequence as the weight producer and adds the input boxes to every stage, but only
// after the consumers have passed the op's barrier: unlike weights, activations are the
// previous op's output.
__device__ __noinline__ void xproducer_loop(Ctx& c) {
  const KParams& p = c.p;
  if (p.x_rows == 0) return;
  const int S = p.num_stages;
  volatile int* fl = c.flags();
  int s = 0;
  uint32_t empty_parity = 1;
  unsigned lin_seq = 0;
  unsigned issued_mask = 0, xphase = 0;  // per stage: boxes issued; parity of the stage's next box phase
  const uint32_t bar_x0 = c.xfull_bar(0), bar_empty0 = c.empty_bar(0);
  const uint32_t x_sub = (uint32_t)p.x_rows * 128u;
  for (int iter = 1;; ++iter) {
    int go;
    {
      unsigned long long t0 = 0;
      int spins = 0;
      while (true) {
        go = fl[0];
        if (go < 0 || (go >> 8) >= iter) break;
        __nanosleep(40);
        if (((++spins) & 255) == 0) {
          if (aborted(c)) { go = -1; break; }
          const unsigned long long now = globaltimer();
          if (t0 == 0) t0 = now;
          if (now - t0 > 4 * c.p.timeout_ns) { go = -1; break; }
        }
      }
    }
    if (go < 0) break;
    const int T = go & 255;
    bool dead = false;
    for (int oi = 0; oi < p.num_ops && !dead; ++oi) {
      const OpDesc& op = p.ops[oi];
      if (op.type != OP_LINEAR) continue;
      lin_seq += 1;
      if (op.flags & F_ROWS) {
        const unsigned n = rows_stage_count(op) * (unsigned)linear_passes(op, T);
        for (unsigned i = 0; i < n; ++i)
          if (++s == S) { s = 0; empty_parity ^= 1u; }
        continue;
      }
      TileCursor lc;
      if (!cursor_open(p, lc, oi)) continue;
      if (!(op.flags & F_XTILE)) {
        // stages of this op carry no activation boxes, but they advance the ring
        const unsigned n = (lc.t1 - lc.tile) * (unsigned)linear_passes(op, T);
        for (unsigned i = 0; i < n; ++i)
          if (++s == S) { s = 0; empty_parity ^= 1u; }
        continue;
      }
      // wait until the consumers have passed this op's barrier
      {
        unsigned long long t0 = 0;
        int spins = 0;
        while ((unsigned)fl[4] < lin_seq) {
          if (fl[0] < 0) { dead = true; break; }
          __nanosleep(64);  // a hot spin would take issue slots from the consumer warps of this scheduler
          if (((++spins) & 1023) == 0) {
            if (aborted(c)) { dead = true; break; }
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            if (now - t0 > 4 * c.p.timeout_ns) { dead = true; break; }
          }
        }
      }
      if (dead) break;
      const int passes = linear_passes(op, T);
      const unsigned t0 = lc.tile;
      for (int g = 0; g < passes && !dead; ++g) {
        if (g > 0) cursor_open(p, lc, oi);
        for (unsigned tile = t0; tile < lc.t1; ++tile) {
          if (!mbar_wait(c, bar_empty0 + 8 * s, empty_parity, ST_TIMEOUT_EMPTY)) {
            dead = true;
            break;
          }
          const uint32_t full = bar_x0 + 8 * s;
          const uint32_t dst = c.smem_addr + (uint32_t)s * (uint32_t)p.stage_bytes + kStageBytes;
          mbar_arrive_expect_tx(full, 2 * x_sub);
          tma_load_2d(dst, op.tmap_x, full, lc.kt * kTileK, g * op.aux3);
          tma_load_2d(dst + x_sub, op.tmap_x, full, lc.kt * kTileK + kBoxK, g * op.aux3);
          issued_mask |= 1u << s;
          xphase ^= 1u << s;
          if (++s == S) { s = 0; empty_parity ^= 1u; }
          if (++lc.kt == lc.nkt) { lc.kt = 0; lc.blk += 1; }
        }
      }
    }
    if (dead || p.mode == MODE_ONEPASS) break;
  }
  // no copy of this thread may still be in flight when the CTA exits
  for (int i = 0; i < S; ++i)
    if (issued_mask & (1u << i)) mbar_wait(c, bar_x0 + 8 * i, ((xphase >> i) & 1u) ^ 1u, ST_TIMEOUT_FULL);
}

// ------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------
template <int PATH>
__global__ void __launch_bounds__(kNumThreads, 1) megakernel(const __grid_constant__ KParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Ctx c(p);
  // 128-byte-swizzled TMA stages need a 1024-byte-aligned base; the host budgets the slack
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  c.smem = smem_raw + pad;
  c.smem_addr = raw_addr + pad;
  c.epoch = p.bar_epoch0;
#if MK_HIER_BARRIER
  c.nbar = 0;
  c.cl_size = p.cluster > 1 ? (uint32_t)p.cluster : 1u;
  c.cl_rank = 0;
  if (c.cl_size > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(c.cl_rank));
#endif
  c.cons_idx = 0;
  c.xphase = 0;
  c.arrived = false;
  c.attn_iter = -1;
  c.tmem = 0u;
  c.has_tmem = false;
  c.done_phase = 0;
  c.tid = threadIdx.x;
  c.lane = threadIdx.x & 31;
  c.warp = threadIdx.x >> 5;
  c.iter = 0;
  c.cur_op = -1;
  c.dbg = nullptr;
  c.pr = nullptr;
  c.dead = false;
  c.ar_seq = 0;
  c.lin_seq = 0;
  volatile int* fl = c.flags();
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; ++s) {
      mbar_init(c.full_bar(s), 1);
      mbar_init(c.empty_bar(s), kNumConsumerWarps);
      mbar_init(c.xfull_bar(s), 1);
    }
    mbar_init(c.done_bar(), 1);
#if MK_HIER_BARRIER
    mbar_init(c.cl_arrive_bar(), c.cl_size);
    mbar_init(c.cl_open_bar(), 1);
#endif
    fl[0] = 0;
    fl[1] = 0;
    fl[2] = 0;
    fl[3] = 0;
    fl[4] = 0;
    fl[5] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
#if MK_HIER_BARRIER
  if (c.cl_size > 1) {  // no CTA may arrive on a peer's mbarrier before it is initialised
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
#endif
  // Tensor memory for the tcgen05 linears (32 or 64 token rows per box): x_rows columns of fp32
  // accumulators, allocated once by warp 0 and freed by it when the CTA leaves.
  constexpr bool use_tmem = PATH == PATH_UMMA;
  if (use_tmem) {
    if (c.warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c.tmem_slot()), "r"((uint32_t)p.x_rows) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    c.tmem = *reinterpret_cast<volatile uint32_t*>(c.smem + p.bar_off + 24 * p.num_stages + 72);
    c.has_tmem = true;
  }

  if (c.warp == kNumConsumerWarps) {
    if (c.lane == 0) producer_loop<PATH>(c);
    __syncwarp();
  } else if (c.warp == kNumConsumerWarps + 1) {
    if constexpr (PATH == PATH_ROWS) {
      rows_prefetch_loop(c);
    } else {
      if (c.lane == 0) xproducer_loop(c);
    }
    __syncwarp();
  } else {
    for (int iter = 1;; ++iter) {
      c.iter = iter;
      c.cur_op = -1;
      int T;
      unsigned long long* prof = p.prof;
      if (prof && c.tid == 0) prof[((size_t)p.num_ops * gridDim.x + blockIdx.x) * 4 + 0] = globaltimer();
      if (p.mode == MODE_OFFLINE) {
        if (blockIdx.x == 0) {
          consumer_sync();
          if (c.tid == 0) {
            int n = 0;
            const int done_before = p.sched[7];  // iterations completed by earlier kernels of this generation call
            const int git = done_before + iter;  // this iteration's number within the call
            bool hand_over = false;
            if (!aborted(c)) {
              if (iter == 1 && p.sched[5] > 0) {
                // prepared by the kernel that handed this iteration over
                n = p.sched[5];
                p.sched[5] = 0;
              } else {
                // sched[4] != 0: the last iteration's outputs have not been appended yet
                if (p.sched[4] != 0) bookkeep_finish(c);
                p.sched[4] = 0;
                if (p.max_iters == 0 || git <= p.max_iters) {
                  n = bookkeep_prepare(c);
                  if (n > 0) p.sched[4] = 1;
                }
              }
              if (n > 0 && (n < p.tok_lo || n > p.tok_hi)) {
                // not an iteration for this program: leave it prepared and let the host launch the other one
                p.sched[5] = n;
                p.sched[7] = git - 1;
                hand_over = true;
              }
            }
            if (!hand_over && git - 1 < p.max_step_times) {
              p.step_times[2 * (git - 1)] = globaltimer();
              p.step_times[2 * (git - 1) + 1] = (unsigned long long)n;
            }
            p.sched[3] = git - 1;
            p.ctrl[0] = hand_over ? -2 : (n > 0 ? n : -1);
            __threadfence();
          }
        }
        grid_sync(c);
        T = __ldcg(p.ctrl);
      } else {
        T = (iter == 1) ? __ldcg(p.qo_indptr + p.max_reqs) : -1;
        if (T == 0) T = -1;
      }
      if (aborted(c)) T = -1;
      // the whole CTA must agree: take thread 0's view
      if (c.tid == 0) fl[3] = T;
      consumer_sync();
      T = fl[3];
      consumer_sync();
      if (prof && c.tid == 0) prof[((size_t)p.num_ops * gridDim.x + blockIdx.x) * 4 + 2] = globaltimer();
      if (T <= 0) break;
      if (T > 255) T = 255;
      if (c.tid == 0) fl[0] = (iter << 8) | T;

      // The op descriptors are read from a two-slot copy in shared memory: the next op's
      // descriptor is fetched asynchronously while the current op runs, so that no op starts
      // with a round trip to L2 for its own parameters.
      constexpr int kDescVecs = (int)(sizeof(OpDesc) / 16);
      OpDesc* sdesc = reinterpret_cast<OpDesc*>(c.smem + p.bar_off + 512);
      if (c.tid < kDescVecs)
        reinterpret_cast<uint4*>(&sdesc[0])[c.tid] = __ldg(reinterpret_cast<const uint4*>(&p.ops[0]) + c.tid);
      for (int oi = 0; oi < p.num_ops; ++oi) {
        if (c.tid < kDescVecs) asm volatile("cp.async.wait_all;" ::: "memory");
        consumer_sync();
        const OpDesc& op = sdesc[oi & 1];
        if (oi + 1 < p.num_ops && c.tid < kDescVecs) {
          const uint32_t dst = smem_u32(&sdesc[(oi + 1) & 1]) + 16 * c.tid;
          const void* src = reinterpret_cast<const uint4*>(&p.ops[oi + 1]) + c.tid;
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
          asm volatile("cp.async.commit_group;" ::: "memory");
        }
        c.cur_op = oi;
        unsigned long long* pr = prof ? prof + ((size_t)oi * gridDim.x + blockIdx.x) * 4 : nullptr;
        c.dbg = (prof && oi == p.trace_op) ? prof + ((size_t)(p.num_ops + 1) * gridDim.x) * 4 + (size_t)blockIdx.x * 16 : nullptr;
        if (pr && c.tid == 0) pr[0] = globaltimer();
        c.pr = pr;
        c.dead = false;
        if ((op.flags & F_CTA0_ONLY) && blockIdx.x != 0) {
          if (op_barrier(c, op)) break;
          if (pr && c.tid == 0) pr[2] = pr[1];
          continue;
        }
        switch (op.type) {
          case OP_EMBED: if (!op_barrier(c, op)) op_embed(c, op, T); break;
          case OP_RMSNORM: op_rmsnorm(c, op, T); break;
          case OP_LINEAR: op_linear<PATH>(c, op, T); break;
          case OP_ATTN:
            op_attention<PATH>(c, op, T);
            break;
          case OP_SILU_MUL: if (!op_barrier(c, op)) op_silu_mul(c, op, T); break;
          case OP_ARGMAX_PARTIAL: if (!op_barrier(c, op)) op_argmax_partial(c, op, T); break;
          case OP_ARGMAX_REDUCE: if (!op_barrier(c, op)) op_argmax_reduce(c, op, T); break;
          case OP_ALLREDUCE: op_allreduce(c, op, T); break;
#if MK_WITH_MOE
          case OP_MOE_ROUTE: if (!op_barrier(c, op)) op_moe_route(c, op, T); break;
          case OP_MOE_LINEAR: op_moe_linear(c, op, T); break;
          case OP_MOE_COMBINE: if (!op_barrier(c, op)) op_moe_combine(c, op, T); break;
#endif
          default: op_barrier(c, op); break;
        }
        if (pr && c.tid == 0) pr[2] = globaltimer();
        if (c.dead) break;
      }
      if (p.mode == MODE_ONEPASS) break;
      if (aborted(c)) {
        // fall through to the next iteration's uniform abort check
      }
    }
    // the producer may be waiting for the next iteration
    consumer_sync();
    if (c.tid == 0) {
      fl[0] = -1;
      // exchanges executed by this launch: the host advances its running sequence base by it
      if (blockIdx.x == 0) p.sched[6] = (int)c.ar_seq;
    }
  }
  __syncthreads();
  // no CTA may exit with a bulk copy still writing its shared memory
  if (threadIdx.x == 0) {
    const unsigned issued = (unsigned)fl[1];
    for (unsigned i = c.cons_idx; i < issued; ++i)
      mbar_wait(c, c.full_bar(i % p.num_stages), (i / p.num_stages) & 1, ST_TIMEOUT_FULL);
  }
  __syncthreads();
  if (use_tmem && c.warp == 0) {
    // every tensor-core operation of this CTA has completed before its columns are given back:
    // one more commit collects whatever an aborted pass left in flight (bounded wait)
    if (c.lane == 0) {
      umma_commit(c.done_bar());
      mbar_wait(c, c.done_bar(), c.done_phase & 1u, ST_TIMEOUT_FULL);
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(c.tmem), "r"((uint32_t)p.x_rows) : "memory");
  }
#if MK_HIER_BARRIER
  if (c.cl_size > 1) {  // a peer may still be storing into this CTA's shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
#endif
}

}  // namespace MK_VARIANT

#ifndef MK_VARIANT_SECONDARY
__global__ void init_state_kernel(KParams p) {
  const int tid = threadIdx.x + blockIdx.x * blockDim.x;
  const int nth = blockDim.x * gridDim.x;
  for (int i = tid; i < p.total_requests; i += nth) p.step[i] = 0;
  for (int i = tid; i < p.max_reqs; i += nth) p.request_ids[i] = -1;
  for (int i = tid; i <= p.max_reqs; i += nth) {
    p.qo_indptr[i] = 0;
    p.kv_indptr[i] = 0;
  }
  for (int i = tid; i < p.max_pages; i += nth) p.page_queue[i] = i;
  if (tid == 0) {
    p.sched[0] = 0;
    p.sched[1] = p.max_pages;
    p.sched[2] = 0;
    p.sched[3] = 0;
    p.sched[4] = 0;
    p.sched[5] = 0;
    p.sched[6] = 0;
    p.sched[7] = 0;
  }
}

#endif
}  // namespace mk

#define MK_CAT2(a, b) a##b
#define MK_CAT(a, b) MK_CAT2(a, b)

#ifdef MK_VARIANT_SECONDARY
// a secondary build only exports its kernel instances
extern "C" const void* MK_CAT(mk_kernel_variant_, MK_VARIANT)(int path) {
  switch (path) {
    case mk::PATH_ROWS: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_ROWS>;
    case mk::PATH_UMMA: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_UMMA>;
    default: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_TILES>;
  }
}
#else
// ------------------------------------------------------------------------------------
// host-side launch helpers (called by the runtime in mk_runtime.cpp)
// ------------------------------------------------------------------------------------
extern "C" const void* mk_kernel_variant_tp(int path);
extern "C" const void* mk_kernel_variant_hier(int path);
extern "C" const void* mk_kernel_variant_moe(int path);
namespace {
// the build of the kernel a launch needs: tensor-parallel exchange code only when there are peers,
// the hierarchical barrier only when the launch uses clusters
const void* kernel_for(const mk::KParams* p) {
  if (p->has_moe) return mk_kernel_variant_moe(p->path);
  if (p->cluster > 1) return mk_kernel_variant_hier(p->path);
  if (p->world > 1) return mk_kernel_variant_tp(p->path);
  switch (p->path) {
    case mk::PATH_ROWS: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_ROWS>;
    case mk::PATH_UMMA: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_UMMA>;
    default: return (const void*)mk::MK_VARIANT::megakernel<mk::PATH_TILES>;
  }
}
}  // namespace

extern "C" int mk_kernel_max_ctas_per_sm(const mk::KParams* p, int smem_bytes) {
  int n = 0;
  const void* k = kernel_for(p);
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, mk::kNumThreads, smem_bytes) != cudaSuccess) return -1;
  return n;
}

// Clusters of `cluster` CTAs that can be resident at once (the hierarchical barrier needs all of them).
extern "C" int mk_kernel_max_clusters(int path, int smem_bytes, int cluster, int grid) {
  const void* k = mk_kernel_variant_hier(path);
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(mk::kNumThreads);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, k, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}

extern "C" int mk_kernel_launch(const mk::KParams* p, int grid, int smem_bytes, void* stream) {
  const void* k = kernel_for(p);
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  void* args[] = {(void*)p};
  if (p->cluster <= 1) {
    e = cudaLaunchCooperativeKernel(k, dim3(grid), dim3(mk::kNumThreads), args, (size_t)smem_bytes, (cudaStream_t)stream);
    return (int)e;
  }
  // co-resident grid of thread-block clusters
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(mk::kNumThreads);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = p->cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeCooperative;
  at[1].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  e = cudaLaunchKernelExC(&cfg, k, args);
  return (int)e;
}

extern "C" int mk_kernel_init_state(const mk::KParams* p, void* stream) {
  mk::init_state_kernel<<<4, 256, 0, (cudaStream_t)stream>>>(*p);
  return (int)cudaGetLastError();
}
#endif  // MK_VARIANT_SECONDARY
