// One decode token of a Llama-architecture model as ONE kernel: every layer's
// rms_norm -> Q/K/V -> RoPE + KV store -> attention -> output projection + residual ->
// rms_norm -> gate/up -> SwiGLU -> down projection + residual
// (src/emel/text/generator/detail.hpp:3746-3840 compute_layer_attention_residual,
//  :3852-3926 compute_layer_feed_forward) runs inside a persistent grid of one CTA per
// SM.  What a chain of per-operation launches pays per launch — the drain of the
// machine, the dependency hand-over, the ramp-up of the next kernel's copies — is paid
// here as one grid barrier per phase (five per layer), and the weights keep streaming
// across the barriers: the weight bytes of a token are known before it starts, so one
// producer warp per CTA walks the CTA's whole list of weight tiles, phase after phase,
// layer after layer, and refills a consumer warp's two stages as soon as that warp
// hands them back — barriers gate the arithmetic, never the copies.  (With the copies
// issued by the consumer warps themselves, a warp spent about as long blocked on the
// issue of its next tile — the memory system's back-pressure — as on the arithmetic.)
//
// The arithmetic is the library's own, piece by piece: gemv4_core.cuh for the Q4_K
// products (bit-identical to the reference's x86 route), attention_core.cuh for the
// split-KV attention (same bits as the stand-alone split + merge kernels), the shared
// quantizer and exact-expf bodies for what sits between them.  Compiled with
// -fmad=false.
//
// Layout of a product phase: a fill = 4 rows x up to two 2048-weight chunks, the unit a
// consumer warp's two stages hold.  A task is one fill (or two: the same four rows of the
// gate and of the up matrix, so the warp that owns them applies SwiGLU itself).  The
// CTA takes the tasks t = blockIdx, blockIdx + grid, ... of every phase and deals them to
// its 16 consumer warps in turn, counting on across phases.  A row whose K spans several
// chunk pairs is completed through the block-value table by the warp that arrives last
// (gemv4_core.cuh).  Attention: a 4-warp group takes one (KV head, query-head quad, KV
// range) unit at a time; the group that delivers the last range of a quad merges the
// ranges and writes the result quantized for the output projection.
//
// Every wait is bounded (mbarrier polls, the grid barrier); a wait that runs out raises
// the status word and the abort flag, every CTA leaves at its next barrier, and a warp
// that leaves first waits (bounded) for the copies still addressed to its stages.
#include "attention_core.cuh"
#include "expf_exact.h"
#include "gemv4_core.cuh"

namespace emelb {

namespace {

using namespace g4;

constexpr int kConsumers = 16;                 // consumer warps 0..15
constexpr int kProducers = 4;                  // producer warps 16..19: batches of four fills, dealt in turn
constexpr int kThreads = (kConsumers + kProducers) * 32;
constexpr int kStageBytes = 4 * CB;            // one slot of the ring: 4 rows x one 2048-weight chunk
constexpr int kSlots = 32;                     // two per consumer warp: the one it works on and one in flight
constexpr int kAttnLmax = 512;                 // KV positions per attention unit
constexpr int kAttnNrep = 2;                   // query heads per unit (the results do not depend on it)
constexpr int kAttnGroupFloats = kAttnNrep * kAttnLmax + 4 * kAttnNrep + kAttnNrep * fa::kMergeMaxSplits + kAttnNrep;
constexpr unsigned long long kBarrierNs = 4000000000ull;   // 4 s
constexpr unsigned long long kDrainNs = 50000000ull;       // 50 ms

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// the 512 consumer threads (the producer warps never join)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 5, 512;" ::: "memory"); }
struct ConsumerSync {
  __device__ __forceinline__ void operator()() const { consumer_sync(); }
};

// bar = {arrivals, generation, abort}.  Called by the consumer threads; returns false (to all of them) when
// the grid is being abandoned: a wait ran out somewhere, here or in another CTA.
// `gen` = the generation this barrier closes (thread 0 reads it once when the kernel starts and counts on).
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned nblocks, volatile int* s_flag, int* status, unsigned& gen_ref) {
  consumer_sync();
  if (threadIdx.x == 0) {
    bool ok = true;
    const unsigned gen = gen_ref++;
    __threadfence();
    const unsigned old = atomicAdd(bar, 1u);
    if (old == nblocks - 1) {
      atomicExch(bar, 0u);
      __threadfence();
      st_release_gpu(bar + 1, gen + 1);
    } else {
      unsigned long long t0 = 0;
      unsigned polls = 0;
      while (ld_acquire_gpu(bar + 1) == gen) {
        if ((++polls & 63u) == 0) {
          if (ld_relaxed_gpu(bar + 2) != 0) { ok = false; break; }
          const unsigned long long now = now_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > kBarrierNs) {
            ok = false;
            atomicExch(bar + 2, 1u);
            if (status) atomicExch(status, 1);
            break;
          }
        }
      }
    }
    if (ld_relaxed_gpu(bar + 2) != 0) ok = false;
    *s_flag = ok ? 1 : 0;
  }
  consumer_sync();
  return *s_flag != 0;
}

// ---------------------------------------------------------------- phases, tasks, fills
enum { PH_QKV = 0, PH_WO = 1, PH_GU = 2, PH_DOWN = 3 };

// (named fields and selects instead of small arrays: a run-time index would put them in local memory)
struct Phase {
  const uint8_t *w0, *w1, *w2;
  int m0, m1, m2;
  int ng0, ng1, ng2;   // 4-row groups per matrix
  int K, nchunks, nsc, ntasks;
  int kind;
  bool paired;         // gate/up with the whole row in one fill: a task = the gate fill, then the up fill
  int64_t row_bytes;
  __device__ __forceinline__ const uint8_t* W(int seg) const { return seg == 0 ? w0 : (seg == 1 ? w1 : w2); }
  __device__ __forceinline__ int M(int seg) const { return seg == 0 ? m0 : (seg == 1 ? m1 : m2); }
};

__device__ __forceinline__ Phase make_phase(int kind, const uint8_t* w0, int m0, const uint8_t* w1, int m1, const uint8_t* w2,
                                            int m2, int K) {
  Phase ph;
  ph.kind = kind;
  ph.w0 = w0; ph.w1 = w1; ph.w2 = w2;
  ph.m0 = m0; ph.m1 = m1; ph.m2 = m2;
  ph.ng0 = (m0 + 3) >> 2; ph.ng1 = (m1 + 3) >> 2; ph.ng2 = (m2 + 3) >> 2;
  ph.K = K;
  ph.nchunks = K / CHUNK;
  ph.nsc = (ph.nchunks + 1) >> 1;
  ph.paired = kind == PH_GU && ph.nsc == 1;
  // gate/up: rows of the two matrices are always taken group by group together (m0 == m1)
  ph.ntasks = kind == PH_GU ? (ph.paired ? ph.ng0 : ph.ng0 * 2 * ph.nsc) : (ph.ng0 + ph.ng1 + ph.ng2) * ph.nsc;
  ph.row_bytes = (int64_t)(K / QK_K) * Q4_K_BYTES;
  return ph;
}

__device__ __forceinline__ Phase layer_phase(const TokenArgs& p, const TokenLayerW& w, int kind) {
  const int qd = p.heads * p.head_dim, kvd = p.kv_heads * p.head_dim;
  switch (kind) {
    case PH_QKV: return make_phase(kind, w.wq, qd, w.wk, kvd, w.wv, kvd, p.n_embd);
    case PH_WO: return make_phase(kind, w.wo, p.n_embd, nullptr, 0, nullptr, 0, qd);
    case PH_GU: return make_phase(kind, w.gate, p.n_ff, w.up, p.n_ff, nullptr, 0, p.n_embd);
    default: return make_phase(kind, w.down, p.n_embd, nullptr, 0, nullptr, 0, p.n_ff);
  }
}

struct Fill {
  int seg, gl, grp, sc, nch;   // matrix, 4-row group inside it, table group (and counter), chunk pair, chunks in it
};

// fill f (0, or 1 for the up half of a paired task) of task t
__device__ __forceinline__ Fill decode_fill(const Phase& ph, int t, int f) {
  Fill k;
  if (ph.kind == PH_GU) {
    if (ph.paired) {
      k.seg = f; k.gl = t; k.grp = t; k.sc = 0;
    } else {
      const int per = 2 * ph.nsc, pg = t / per, rem = t - pg * per;
      k.seg = rem >= ph.nsc ? 1 : 0;
      k.sc = rem - k.seg * ph.nsc;
      k.gl = pg; k.grp = pg;           // table group = the 8 rows {gate rows, up rows} of group pg
    }
  } else {
    const int g_all = t / ph.nsc;
    k.sc = t - g_all * ph.nsc;
    k.seg = g_all < ph.ng0 ? 0 : (g_all < ph.ng0 + ph.ng1 ? 1 : 2);
    k.gl = g_all - (k.seg == 0 ? 0 : (k.seg == 1 ? ph.ng0 : ph.ng0 + ph.ng1));
    k.grp = g_all;
  }
  k.nch = min(2, ph.nchunks - 2 * k.sc);
  return k;
}

// tasks of a phase that belong to CTA b of G
__device__ __forceinline__ int cta_tasks(const Phase& ph, int b, int G) { return b < ph.ntasks ? (ph.ntasks - b + G - 1) / G : 0; }

struct Ring {
  uint32_t ring0;   // shared address of the CTA's slots
  uint32_t full0;   // per slot one mbarrier: the chunk's bytes have landed
  uint32_t empty0;  // per slot one mbarrier: the consumer is done with it
  unsigned task;    // the task this warp holds (numbered across phases)
};

}  // namespace

// ---------------------------------------------------------------- producer warps
// The CTA's chunks (4 rows x 2048 weights) are numbered in the order the consumers take them — across tasks,
// phases and layers — and chunk m lives in slot m % 32 of the CTA's ring.  Every slot has one owner for the
// whole kernel: four lanes (one per row) of a producer warp, which walk the slot's chunks m = slot, slot + 32,
// ... on their own and refill the slot as soon as a consumer warp hands it back; the 32 walkers of the four
// producer warps share each warp's instruction stream but never wait for one another.  (One owner per slot
// also keeps the parity waits sound: a slot's uses are issued in order by the same lanes.)  Every task takes
// the same number of slots in its phase (a chunk pair with one chunk leaves its second slot empty: the owner
// completes that slot's barrier phase without a copy), so slot and barrier parity follow from m alone.
// armed[s] (shared): chunk number + 1 last issued to slot s; *done: counts the producers that have left.
__device__ __forceinline__ void run_producer(const TokenArgs& p, uint32_t ring0, uint32_t full0, uint32_t empty0, volatile int* armed,
                                             int* done, int lane, int pw) {
  const int G = gridDim.x, b = blockIdx.x;
  const int slot = 8 * pw + (lane >> 2), r = lane & 3;
  const uint32_t stage = ring0 + slot * kStageBytes, full = full0 + 8 * slot, bar = empty0 + 8 * slot;
  unsigned m = slot;          // this walker's next chunk
  unsigned M = 0;             // chunks before the walker's current phase
  uint32_t use = 0;           // times the slot has been filled
  int l = 0, kind = PH_QKV;
  Phase ph = layer_phase(p, p.layers[0], PH_QKV);
  unsigned total = cta_tasks(ph, b, G) * (ph.paired ? 4 : 2);
  bool active = true, ready = false, copy = false, ok = true;
  const uint8_t* src = nullptr;
  unsigned polls = 0;
  unsigned long long t0 = 0;
  while (__any_sync(0xffffffffu, active)) {
    if (active && !ready) {
      // the phase that holds chunk m, then the chunk's place in it
      while (m >= M + total) {
        M += total;
        if (++kind > PH_DOWN) { kind = PH_QKV; ++l; }
        if (l >= p.n_layer) { active = false; break; }
        ph = layer_phase(p, p.layers[l], kind);
        total = cta_tasks(ph, b, G) * (ph.paired ? 4 : 2);
      }
      if (active) {
        const int idx = (int)(m - M);
        const int j = ph.paired ? idx >> 2 : idx >> 1, i = idx & (ph.paired ? 3 : 1), f = i >> 1, ci = i & 1;
        const Fill k = decode_fill(ph, b + j * G, f);
        copy = ci < k.nch;
        const int row = min(k.gl * 4 + r, ph.M(k.seg) - 1);
        src = ph.W(k.seg) + (size_t)row * ph.row_bytes + (size_t)(2 * k.sc + ci) * CB;
        ready = true;
      }
    }
    // a fresh barrier passes a wait on parity 1: the first fill does not wait
    if (active && ready && mbar_try_wait(bar, (use & 1u) ^ 1u)) {
      if (r == 0) {
        armed[slot] = (int)m + 1;
        if (copy) mbar_expect_tx(full, 4 * CB);
        else mbar_arrive(full);                    // no chunk for this slot: its phase completes empty
      }
      if (copy) bulk_g2s(stage + r * CB, src, CB, full);
      m += kSlots;
      ++use;
      ready = false;
      polls = 0;
      t0 = 0;
    }
    if (active && (++polls & 255u) == 0) {
      if (ld_relaxed_gpu(p.bar + 2) != 0) ok = false;
      const unsigned long long now = now_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kBarrierNs) ok = false;
    }
    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
  }
  if (!ok && lane == 0) {
    atomicExch(p.bar + 2, 1u);
    if (p.status) atomicExch(p.status, 1);
  }
  __syncwarp();
  if (lane == 0) {
    __threadfence_block();
    atomicAdd(done, 1);
  }
}

// ---------------------------------------------------------------- consumer side of a product phase
// The CTA's tasks of `ph` against the activation vector at shared address A.  The consumer warps take the
// CTA's tasks in order from a shared counter (ring.task = the task this warp holds, numbered across phases;
// tbase / mbase = tasks / fills of the earlier phases).  Returns false when a copy wait ran out.
__device__ __forceinline__ bool run_phase(const TokenArgs& p, const Phase& ph, Ring& ring, uint32_t A, int lane, unsigned tbase,
                                          unsigned mbase, int* s_task, volatile int* armed, volatile int* s_done, int layer) {
  const int G = gridDim.x, b = blockIdx.x;
  const int nt = cta_tasks(ph, b, G), nf = ph.paired ? 2 : 1;
  while (ring.task < tbase + nt) {
    const int j = (int)(ring.task - tbase);
    const int t = b + j * G;
    float gate_sum = 0.0f;
    for (int f = 0; f < nf; ++f) {
      const Fill k = decode_fill(ph, t, f);
      float bv0 = 0.0f, bv1 = 0.0f;
      for (int ci = 0; ci < 2; ++ci) {
        const unsigned m = mbase + j * (2 * nf) + 2 * f + ci;
        const int slot = m & (kSlots - 1);
        const uint32_t use = m / kSlots;
        // A parity wait tells the current barrier phase from the previous one only, and a warp may hold a chunk
        // that is more than one turn of the ring ahead of the slot's state: first wait until the producer has
        // armed the slot for exactly this chunk.
        bool ok = true;
        if (lane == 0) {
          unsigned polls = 0;
          unsigned long long t0 = 0;
          while (armed[slot] != (int)m + 1) {
            if ((++polls & 255u) == 0) {
              const unsigned long long now = now_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > kWaitNs) { ok = false; break; }
            }
          }
        }
        if (!__all_sync(0xffffffffu, ok)) return false;
        ok = mbar_wait_bounded(ring.full0 + 8 * slot, use & 1u);
        if (!__all_sync(0xffffffffu, ok)) return false;
        if (ci < k.nch) {
          float one[1];
          q4k_item<1>(ring.ring0 + slot * kStageBytes, A, ph.K, (2 * k.sc + ci) * 8 + (lane & 7), lane, one);
          if (ci == 0) bv0 = one[0];
          else bv1 = one[0];
        }
        __syncwarp();
        if (lane == 0) {
          s_done[slot] = (int)m + 1;
          mbar_arrive(ring.empty0 + 8 * slot);    // the slot goes back to the producers
        }
      }
      float sum = 0.0f;
      bool done;
      if (ph.nsc == 1) {
        // the whole row is in this fill: ascending block order inside the warp
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv0, (lane & ~7) + i));
        if (k.nch == 2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv1, (lane & ~7) + i));
        }
        sum = __shfl_sync(0xffffffffu, acc, (lane & 3) * 8);   // lane j < 4: row j of the group
        done = true;
      } else if (ph.kind == PH_GU) {
        // 8-row table groups {4 gate rows, 4 up rows}; the last of the 2 * nsc fills sums all eight
        const int r4 = lane >> 3, bb = lane & 7, nblk = ph.nchunks * 8;
        float* rows = p.bv_table + ((size_t)k.grp * 8 + k.seg * 4 + r4) * nblk + bb;
        __stcg(rows + (2 * k.sc) * 8, bv0);
        if (k.nch == 2) __stcg(rows + (2 * k.sc + 1) * 8, bv1);
        done = arrive_group<2>(p.bv_table, p.grp_cnt, k.grp, 2 * ph.nsc, ph.nchunks, lane, sum);
      } else {
        const float one0[1] = {bv0};
        store_item<1>(one0, p.bv_table, k.grp, 2 * k.sc, ph.nchunks, lane);
        if (k.nch == 2) {
          const float one1[1] = {bv1};
          store_item<1>(one1, p.bv_table, k.grp, 2 * k.sc + 1, ph.nchunks, lane);
        }
        done = arrive_group<1>(p.bv_table, p.grp_cnt, k.grp, ph.nsc, ph.nchunks, lane, sum);
      }
      if (!done) continue;
      const int row = k.gl * 4 + lane;
      const bool live = lane < 4 && row < ph.M(k.seg);
      if (ph.kind == PH_QKV) {
        // rows 2p, 2p+1 of a head are one rotation pair (apply_rope_pairing,
        // src/emel/text/generator/detail.hpp:2905-2936; KV rows rounded to f16, :3294-3332)
        const float other = __shfl_xor_sync(0xffffffffu, sum, 1);
        if (live) {
          const int hd = p.head_dim, head = row / hd, d = row - head * hd;
          const int pos = p.state[1];
          float out = sum;
          if (k.seg < 2 && d < p.rope_rot_dim) {
            const int pairs = p.rope_rot_dim >> 1;
            const float cs = p.rope_cos[(int64_t)pos * pairs + (d >> 1)], sn = p.rope_sin[(int64_t)pos * pairs + (d >> 1)];
            out = (d & 1) ? __fadd_rn(__fmul_rn(other, sn), __fmul_rn(sum, cs)) : __fsub_rn(__fmul_rn(sum, cs), __fmul_rn(other, sn));
          }
          if (k.seg == 0) p.q[row] = out;
          else {
            __half* cache = (k.seg == 1 ? p.kcache : p.vcache) + (int64_t)layer * p.kv_heads * p.capacity * hd;
            cache[((int64_t)head * p.capacity + pos) * hd + d] = __float2half_rn(out);
          }
        }
      } else if (ph.kind == PH_GU) {
        // ffn = (gate / (1 + expf(-gate))) * up (silu: src/emel/text/generator/detail.hpp:2967-2973; :3911-3913)
        float g, u;
        if (ph.paired) {
          if (f == 0) { gate_sum = sum; continue; }
          g = gate_sum;
          u = sum;
        } else {
          g = sum;                                        // lanes 0-3: gate rows, lanes 4-7: the same rows of up
          u = __shfl_down_sync(0xffffffffu, sum, 4);
        }
        if (live) p.ffn[row] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), u);
      } else {
        if (live) p.hidden[row] = __fadd_rn(__ldcg(p.hidden + row), sum);
      }
    }
    // the next task nobody has taken yet (it may belong to a later phase: the warp keeps it until then)
    int nx = 0;
    if (lane == 0) nx = atomicAdd(s_task, 1);
    ring.task = (unsigned)__shfl_sync(0xffffffffu, nx, 0);
  }
  return true;
}

// attention of one layer over this CTA's share of the (KV head, query-head quad, KV range) units; gs = this
// 4-warp group's shared scratch
template <int D>
__device__ __forceinline__ void run_attention(const TokenArgs& p, int layer, float* gs, int group, int ngroups_total) {
  const int tid = threadIdx.x & 127, warp4 = tid >> 5, lane = tid & 31;
  const fa::GroupSync sync{1 + (int)(threadIdx.x >> 7)};
  float* s_p = gs;
  float* s_red = gs + kAttnNrep * kAttnLmax;
  float* s_w = s_red + 4 * kAttnNrep;
  float* s_inv = s_w + kAttnNrep * fa::kMergeMaxSplits;
  int* s_last = reinterpret_cast<int*>(s_red);   // reused between the unit and its merge
  FlashArgs a{};
  const int64_t layer_off = (int64_t)layer * p.kv_heads * p.capacity * D;
  a.q = p.q;
  a.k = p.kcache + layer_off;
  a.v = p.vcache + layer_off;
  a.dst = p.attn_f32;
  a.k_nb1 = a.v_nb1 = 2 * D;
  a.k_nb2 = a.v_nb2 = 2 * p.capacity * D;
  a.head_dim = D;
  a.heads = p.heads;
  a.kv_heads = p.kv_heads;
  a.scale = p.attn_scale;
  a.splits = p.fa_splits;
  a.part_acc = p.part_acc;
  a.part_ml = p.part_ml;
  const int T = p.state[2];
  const int nz = (p.heads / p.kv_heads) / kAttnNrep;
  const int units = p.kv_heads * nz * p.fa_splits;
  for (int u = group; u < units; u += ngroups_total) {
    const int split = u % p.fa_splits, kz = u / p.fa_splits, z = kz % nz, kh = kz / nz;
    fa::split_unit<D, kAttnNrep, kAttnLmax, 4, true>(a, split, kh, z, T, tid, s_p, s_red, sync);
    // the group that delivers the last range of (kh, z) merges its heads
    __threadfence();
    sync();
    if (tid == 0) {
      const int last = atomicAdd(p.kv_cnt + kz, 1) == p.fa_splits - 1;
      if (last) p.kv_cnt[kz] = 0;
      *s_last = last;
    }
    sync();
    const bool last = *s_last != 0;
    sync();
    if (!last) continue;
    __threadfence();
    const int head0 = kh * (p.heads / p.kv_heads) + z * kAttnNrep;
    if (warp4 < kAttnNrep) fa::merge_head_weights(a, head0 + warp4, lane, s_w + warp4 * fa::kMergeMaxSplits, s_inv + warp4);
    sync();
    float* s_out = s_p;
    {
      // a thread owns VPT of the unit's values: their range walks run side by side
      constexpr int VPT = kAttnNrep * D / 128;
      static_assert((kAttnNrep * D) % 128 == 0 && VPT >= 1, "whole values per thread");
      int hh[VPT], dd[VPT];
      const float* ww[VPT];
      float ii[VPT], oo[VPT];
#pragma unroll
      for (int n = 0; n < VPT; ++n) {
        const int idx = tid + 128 * n, hl = idx / D;
        hh[n] = head0 + hl;
        dd[n] = idx - hl * D;
        ww[n] = s_w + hl * fa::kMergeMaxSplits;
        ii[n] = s_inv[hl];
      }
      fa::merge_outputs<VPT>(a, hh, dd, ww, ii, oo);
#pragma unroll
      for (int n = 0; n < VPT; ++n) {
        s_out[tid + 128 * n] = oo[n];
        if (p.attn_f32) p.attn_f32[(size_t)head0 * D + tid + 128 * n] = oo[n];
      }
    }
    sync();
    // the unit's heads x D values = whole Q8_K blocks of the vector the output projection consumes
    if (warp4 < kAttnNrep * D / QK_K) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s_out[warp4 * QK_K + 8 * lane + i];
      uint32_t lo, hi;
      int bs;
      float dq;
      q8_k_block_warp(v, lane, lo, hi, bs, dq);
      q8_k_store_planes(p.attn_planes, 0, p.heads * D, head0 * D / QK_K + warp4, lane, lo, hi, bs, dq);
    }
    sync();
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) llama_token_kernel(const TokenArgs p) {
  extern __shared__ __align__(16) uint8_t smem_t[];
  __shared__ double s_part[kConsumers];
  __shared__ int s_flag, s_prod_done;
  __shared__ int s_armed[kSlots], s_done[kSlots], s_task;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t base = (s32(smem_t) + 255u) & ~255u;
  uint8_t* A_ptr = smem_t + (base - s32(smem_t));
  const uint32_t A = base;
  const int act_cap = act_bytes(p.n_ff > p.n_embd ? p.n_ff : p.n_embd);
  const uint32_t ring0 = A + act_cap, full0 = ring0 + kSlots * kStageBytes, empty0 = full0 + kSlots * 8;
  float* attn_scratch = reinterpret_cast<float*>(A_ptr + act_cap + kSlots * kStageBytes + kSlots * 16);
  if (threadIdx.x == 0) {
    for (int sl = 0; sl < kSlots; ++sl) {
      mbar_init(full0 + 8 * sl, 1);
      mbar_init(empty0 + 8 * sl, 1);
      s_armed[sl] = 0;
      s_done[sl] = 0;
    }
    s_task = 0;
    s_prod_done = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp >= kConsumers) {
    run_producer(p, ring0, full0, empty0, s_armed, &s_prod_done, lane, warp - kConsumers);
    return;
  }

  Ring ring;
  ring.ring0 = ring0;
  ring.full0 = full0;
  ring.empty0 = empty0;
  {
    int first = 0;
    if (lane == 0) first = atomicAdd(&s_task, 1);
    ring.task = (unsigned)__shfl_sync(0xffffffffu, first, 0);
  }
  unsigned tbase = 0, mbase = 0;
  const int G = gridDim.x;
  const int agroup = (warp >> 2) * G + blockIdx.x, agroups = 4 * G;
  float* my_attn = attn_scratch + (warp >> 2) * kAttnGroupFloats;
  bool alive = true;
  unsigned gen = threadIdx.x == 0 ? ld_acquire_gpu(p.bar + 1) : 0u;   // no barrier of this launch has completed yet
  // phase profile: thread 0 of CTA 0 stamps the nanosecond timer at fixed points of every layer
  auto stamp = [&](int l, int point) {
    if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) p.trace[l * kTokenTracePoints + point] = now_ns();
  };
  // leaving early: the copies still addressed to this warp's stages must land first (bounded)
  auto leave = [&]() {
    const unsigned long long t0 = now_ns();
    while (*(volatile int*)&s_prod_done < kProducers && now_ns() - t0 < kDrainNs) {}
    for (int sl = warp; sl < kSlots; sl += kConsumers) {                 // warp w looks after slots w and w + 16
      const int a = *(volatile int*)&s_armed[sl], d = *(volatile int*)&s_done[sl];
      if (a != 0 && a != d) {
        const uint32_t use = (uint32_t)(a - 1) / kSlots;
        const unsigned long long t1 = now_ns();
        while (!mbar_try_wait(full0 + 8 * sl, use & 1u) && now_ns() - t1 < kDrainNs) {}
      }
    }
  };
  auto fail = [&]() {
    if (lane == 0) {
      atomicExch(p.bar + 2, 1u);
      if (p.status) atomicExch(p.status, 1);
    }
  };

  for (int l = 0; l < p.n_layer; ++l) {
    const TokenLayerW& w = p.layers[l];
    // ---- Q, K, V (hidden is complete: start of the kernel, or the barrier that closed the previous layer)
    stamp(l, 0);
    stage_act_rms_norm<kConsumers>(A_ptr, p.n_embd, p.hidden, w.attn_norm, p.eps, s_part, warp, lane, ConsumerSync{});
    consumer_sync();
    stamp(l, 1);
    {
      const Phase ph = layer_phase(p, w, PH_QKV);
      if (alive && !run_phase(p, ph, ring, A, lane, tbase, mbase, &s_task, s_armed, s_done, l)) { alive = false; fail(); }
      const int nt = cta_tasks(ph, blockIdx.x, G);
      tbase += nt;
      mbase += nt * (ph.paired ? 4 : 2);
    }
    stamp(l, 2);
    if (!grid_barrier(p.bar, G, &s_flag, p.status, gen)) { leave(); return; }

    // ---- attention over the cache rows 0 .. position
    stamp(l, 3);
    run_attention<D>(p, l, my_attn, agroup, agroups);
    stamp(l, 4);
    if (!grid_barrier(p.bar, G, &s_flag, p.status, gen)) { leave(); return; }
    stamp(l, 5);

    // ---- hidden += Wo * attention
    stage_act_planes(A_ptr, p.heads * p.head_dim, p.attn_planes.qs, p.attn_planes.d, p.attn_planes.bsums, threadIdx.x, kConsumers * 32);
    consumer_sync();
    stamp(l, 6);
    {
      const Phase ph = layer_phase(p, w, PH_WO);
      if (alive && !run_phase(p, ph, ring, A, lane, tbase, mbase, &s_task, s_armed, s_done, l)) { alive = false; fail(); }
      const int nt = cta_tasks(ph, blockIdx.x, G);
      tbase += nt;
      mbase += nt * (ph.paired ? 4 : 2);
    }
    stamp(l, 7);
    if (!grid_barrier(p.bar, G, &s_flag, p.status, gen)) { leave(); return; }

    // ---- ffn = swiglu(gate, up) (the SwiGLU is applied by the warp that completes a row of both)
    stamp(l, 8);
    stage_act_rms_norm<kConsumers>(A_ptr, p.n_embd, p.hidden, w.ffn_norm, p.eps, s_part, warp, lane, ConsumerSync{});
    consumer_sync();
    stamp(l, 9);
    {
      const Phase ph = layer_phase(p, w, PH_GU);
      if (alive && !run_phase(p, ph, ring, A, lane, tbase, mbase, &s_task, s_armed, s_done, l)) { alive = false; fail(); }
      const int nt = cta_tasks(ph, blockIdx.x, G);
      tbase += nt;
      mbase += nt * (ph.paired ? 4 : 2);
    }
    stamp(l, 10);
    if (!grid_barrier(p.bar, G, &s_flag, p.status, gen)) { leave(); return; }

    // ---- hidden += Wdown * ffn
    stamp(l, 11);
    stage_act_f32<kConsumers>(A_ptr, p.n_ff, p.ffn, warp, lane);
    consumer_sync();
    stamp(l, 12);
    {
      const Phase ph = layer_phase(p, w, PH_DOWN);
      if (alive && !run_phase(p, ph, ring, A, lane, tbase, mbase, &s_task, s_armed, s_done, l)) { alive = false; fail(); }
      const int nt = cta_tasks(ph, blockIdx.x, G);
      tbase += nt;
      mbase += nt * (ph.paired ? 4 : 2);
    }
    stamp(l, 13);
    if (l + 1 < p.n_layer && !grid_barrier(p.bar, G, &s_flag, p.status, gen)) { leave(); return; }
    stamp(l, 14);
  }
  if (!alive) leave();
}

size_t llama_token_smem_bytes(int n_embd, int n_ff) {
  return 256 + (size_t)g4::act_bytes(n_ff > n_embd ? n_ff : n_embd) + (size_t)kSlots * kStageBytes + kSlots * 16 +
         4 * (size_t)kAttnGroupFloats * sizeof(float);
}

bool llama_token_supported(const TokenArgs& a, int attention_splits, int n_ctx) {
  if (a.head_dim != 128) return false;
  const int n_rep = a.kv_heads > 0 ? a.heads / a.kv_heads : 0;
  if (n_rep <= 0 || n_rep % kAttnNrep != 0 || (kAttnNrep * a.head_dim) % QK_K != 0) return false;
  if (a.n_embd % CHUNK != 0 || a.n_ff % CHUNK != 0 || (a.heads * a.head_dim) % CHUNK != 0) return false;
  if (a.rope_rot_dim > a.head_dim || (a.rope_rot_dim & 1)) return false;
  if (attention_splits < 1 || attention_splits > fa::kMergeMaxSplits || (int64_t)attention_splits * kAttnLmax < n_ctx) return false;
  if (llama_token_smem_bytes(a.n_embd, a.n_ff) > 225 * 1024) return false;
  return true;
}

cudaError_t launch_llama_token(const TokenArgs& a, int sm_count, TokenLaunchState* state, cudaStream_t st) {
  auto kern = llama_token_kernel<128>;
  const size_t smem = llama_token_smem_bytes(a.n_embd, a.n_ff);
  if (state->smem != smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int n = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem);
    if (e != cudaSuccess) return e;
    if (n < 1) return cudaErrorInvalidConfiguration;
    state->smem = smem;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(sm_count);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident at once: the grid barrier depends on it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace emelb
