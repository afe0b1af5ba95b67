// Persistent, warp-specialised, mbarrier-pipelined LoRA shrink / expand kernels (the fast path).
//
// Two CTAs per SM (a grid of 2 x SM count) walk their share of the work items (item i belongs to CTA
// i mod gridDim.x).  The first
// kProducerWarps warps are producers: the 32 lanes of each resolve 32 upcoming items in parallel (tile record ->
// table entries -> row addresses and token ids), then feed a ring of shared-memory stages with bulk asynchronous
// copies (cp.async.bulk + mbarrier complete_tx).  With more than one producer all run the same deterministic
// allocation and stage g is issued by producer g mod kProducerWarps (measured: no gain on B200 while the consumers
// are the bottleneck, so one producer is configured).  The remaining warps are consumers: they wait on a stage's "full" barrier, do the arithmetic and release the
// stage through its "empty" barrier.  Consumer warps never wait for each other (shrink: each warp owns a K-slice and
// the last warp to finish an item, elected by an atomic counter, adds the partial sums; expand: each warp owns a
// 1024-element span of the B chunk), so every wait in the kernel is an mbarrier wait with a time limit.
//
// What shapes the ring (measured on B200): a cp.async.bulk warp-instruction costs the issuing warp 400-600 cycles
// whatever its size and however many lanes take part, and ~1 us passes before the bytes land.  So a stage is filled
// by ONE bulk instruction in which every participating lane carries one copy (adapter rows and activation rows
// alike), stages are made as large as the work item allows (tens of KB), and they are packed back to back in a
// byte ring of kRingBytes so that several are in flight whatever their size.
//
// Programmatic dependent launch: the producer issues the adapter-row copies of the first stages (rows that no kernel
// on the stream writes) before it executes griddepcontrol.wait and stashes the activation copies (x, y, delta) of
// those stages; they go out right after the wait.  With a ring of 96 KB two CTAs fit on an SM: in steady state both
// belong to the running kernel (twice the stages in flight and twice the consumer warps per SM; measured 15 % to
// 38 % less time per layer than one CTA per SM), and as CTAs of the running kernel retire the next kernel's CTAs
// take their place and run their prologue under this kernel's tail.
//
// Shrink stage  = one item (tile, projection, block of <= 4 rows), or a K-chunk of it when the item exceeds
//                 kMaxStageBytes: [nrows adapter-row chunks][n token-row chunks]; accumulators stay in registers
//                 across the chunks of an item.
// Expand stage  = one item (tile, projection, 16384-element chunk of B): [B chunk][n y segments][n delta rows].
//                 y is read through the stage and written back with plain coalesced stores.
#pragma once

#include "lora_common.cuh"

namespace slora {

constexpr int kSlots = 8;  // stage descriptors (barrier pairs) in flight
#ifndef SLORA_RING_KB
#define SLORA_RING_KB 96
#endif
#ifndef SLORA_STAGE_KB
#define SLORA_STAGE_KB 48
#endif
constexpr int kRingBytes = SLORA_RING_KB * 1024;  // ring + control block stay below half an SM's shared memory
#ifndef SLORA_EXPAND_RING_KB
#define SLORA_EXPAND_RING_KB 104
#endif
// The expand's control block is 8 KB smaller (no reduction buffers): with 104 KB three of its ~34 KB stages (a B chunk
// and one token's y segment and delta row) are in flight instead of two.  Used by the EXACT instantiation (long
// launches over mixed ranks: measured -4 % on its q,k,v launch); the short launches of a same-rank decode batch
// measured 2 % slower with it and keep kRingBytes.
constexpr int kExpandRingBytes = SLORA_EXPAND_RING_KB * 1024;
constexpr int kPipeCtasPerSm = 2;      // persistent CTAs per SM
constexpr int kPendSlots = 4;           // stages that may be issued before the grid-dependency wait
constexpr int kProducerWarps = 1;  // stage g is fed by producer warp g % kProducerWarps
constexpr int kConsumerWarps = 8;
constexpr int kPipeThreads = 32 * (kProducerWarps + kConsumerWarps);
constexpr int kMaxStageBytes = SLORA_STAGE_KB * 1024;  // a shrink item is cut into K-chunks no larger than this
constexpr int kPipeChunk = 16384;          // flat B elements per expand item (32 KB)
constexpr int kMaxPieces = 16;  // B copies per expand stage (lanes 0..15); y copies use lanes 16..23, delta 24..31
constexpr int kSpanRows = 6;    // pool rows a B chunk may touch
constexpr int kWideRows = 8;    // adapter rows of a shrink item of a tile with at most kWideTokens tokens (EXACT only)
constexpr int kWideTokens = 4;
constexpr int kCompactTiles = 640;  // tiles whose item counts fit the control block (two CTAs per SM leave little room)

constexpr int FLAG_FIRST = 1, FLAG_LAST = 2, FLAG_END = 4;
constexpr uint32_t FULL_MASK = 0xffffffffu;
constexpr long long kWaitCycles = 400000000ll;  // about 0.2 s of SM clock: far beyond any legitimate wait here

// Wait for a barrier phase for a bounded time (SM cycle counter); false on timeout.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (clock64() - t0 > kWaitCycles) return false;
  }
}

// Shared-memory control block of one pipeline.
struct PipeCtl {
  uint64_t full[kSlots];
  uint64_t empty[kSlots];
  int meta[kSlots][16];
  // one private copy per producer warp of everything below
  struct Prod {
    uint32_t off[kSlots];  // byte offset of each stage in the ring
    // activation copies of the stages issued before the grid-dependency wait (one entry per lane)
    uint64_t pend_src[kPendSlots][32];
    uint32_t pend_dst[kPendSlots][32];
    uint32_t pend_bytes[kPendSlots][32];
    // the 32 items a batch resolves, one per lane, parked here so that the lanes that carry the copies read what
    // they need instead of receiving it through shuffles
    int64_t d_l[32][kWideRows];
    int d_i[32][16];
  } prod[kProducerWarps];
  // planned batches of mixed ranks: items up to and including each tile (see build_item_map)
  uint16_t item_end[kCompactTiles];
  int tp_gave_up;  // in-band signalling: a wait for another rank's values ran out; nobody in this CTA waits again
};

// Shrink only: per-item partial sums of the consumer warps and the arrival counter that elects the last warp.  (Kept
// out of PipeCtl so that the expand, which has no use for it, can give those 8 KB to its ring.)
struct ShrinkRed {
  float sum[kSlots][kConsumerWarps][32];
  int cnt[kSlots];
};

// Producer-side ring state (identical in all 32 lanes).
struct Ring {
  int role = 0;       // which producer warp this is
  uint32_t g = 0;     // next stage index
  uint32_t tail = 0;  // oldest stage not yet known to be released
  uint32_t head = 0;  // next free byte
  bool pre = true;    // still before the grid-dependency wait
  int npend = 0;      // stages with stashed activation copies
  bool dead = false;  // a bounded wait ran out
  uint32_t cap = kRingBytes;  // bytes of the ring
  const TpLink* tp = nullptr;  // expand under tensor parallelism: flags to wait for before activations are read
  int32_t* status = nullptr;
  bool trigger_after_wait = false;  // shrink whose expand starts early: dependents may launch once this has waited
};

constexpr long long kTpLinkWaitCycles = 4000000000ll;  // about 2 s: ranks drift by host-side jitter, not more

// Expand side of the tensor-parallel link: lanes 0..n_parts-1 wait until every rank's columns of this exchange have
// landed in this rank's delta buffer.  Bounded; false when the wait ran out.
__device__ __forceinline__ bool tp_link_wait(const TpLink& tp, int lane) {
  bool seen = true;
  if (lane < tp.n_parts) {
    const int seq = tp.seq_state[tp.half] + 1;
    const int32_t* flag = tp.flags[tp.my_part] + tp.half * tp.n_parts + lane;
    const long long t0 = clock64();
    seen = false;
    while (!seen) {
      int v;
      asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      seen = v >= seq;
      if (!seen && clock64() - t0 > kTpLinkWaitCycles) break;
    }
  }
  return __all_sync(0xffffffffu, seen);
}

// End of a linked launch (whole-launch flags): the last CTA to get here either raises this rank's flag on every rank
// (shrink: all its columns have been written and fenced) or counts the exchange as done (expand: every CTA has read
// its number).  One system-scope fence per CTA, by the thread that then bumps the arrival counter: the CTA barrier
// before it orders every thread's stores before that fence, and a fence is cumulative.  (A fence by each of the CTA's
// 288 threads, as this was first written, serialises in the memory system: measured, it cost more than the exchange
// itself.)  The expand's bookkeeping stays on this GPU and needs no system-scope fence at all.
__device__ __forceinline__ void tp_link_finish(const TpLink& tp, bool is_shrink) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (is_shrink) {
      __threadfence_system();
    } else {
      __threadfence();
    }
    s_last = atomicAdd(tp.counter, 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_last) return;
  const int seq = tp.seq_state[tp.half] + 1;
  if (threadIdx.x == 0) {
    *tp.counter = 0;
    __threadfence();  // the other CTAs' arrivals (device-scope atomics) before what follows
  }
  __syncthreads();
  if (is_shrink) {
    if (static_cast<int>(threadIdx.x) < tp.n_parts) {
      asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(tp.flags[threadIdx.x] + tp.half * tp.n_parts + tp.my_part),
                   "r"(seq)
                   : "memory");
    }
  } else if (threadIdx.x == 0) {
    tp.seq_state[tp.half] = seq;
  }
}

// ---- in-band signalling (TpLink::inband) ------------------------------------------------------------------------
// No flag and no fence at all: the delta buffers start out filled with a bit pattern no result can have (kTpEmpty: a
// NaN that the float-to-16-bit conversion never produces), the shrink stores its results into every rank's buffer
// with plain stores, and the expand checks the delta values themselves: a consumer lane that finds the pattern among
// the eight values it is about to use re-reads them from global memory until they have arrived (bounded).  Each
// 16-bit element is written by one store, so checking every element that is used is enough - no ordering between
// elements is needed.  The last CTA of the expand refills the half it consumed; no rank can write that half again
// before this rank has finished its next exchange on the other half, which starts after this kernel.
constexpr uint32_t kTpEmpty2 = 0xffffffffu;  // two elements of the pattern 0xffff
__device__ __forceinline__ bool tp_has_empty(const uint4& v) {
  // (bitwise ors: no short-circuit branches)
  auto e = [](uint32_t w) { return ((w & 0xffffu) == 0xffffu) | ((w >> 16) == 0xffffu); };
  return (e(v.x) | e(v.y) | e(v.z) | e(v.w)) != 0;
}
// Eight delta values from global memory, polled until none is the empty pattern; false when the wait ran out.
__device__ __forceinline__ bool tp_poll_delta(const void* src, uint4& v, volatile int* gave_up) {
  const long long t0 = clock64();
  for (;;) {
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src)
                 : "memory");
    if (!tp_has_empty(v)) return true;
    if (*gave_up != 0) return false;
    if (clock64() - t0 > kTpLinkWaitCycles) {
      *gave_up = 1;
      return false;
    }
  }
}
// End of an expand with in-band signalling: the last CTA refills the consumed half with the empty pattern.  No fence
// before the arrival: what has to precede the refill is the other CTAs' LOADS of the values, and a load has
// returned its value before the code that follows it (the arrival) runs.
__device__ __forceinline__ void tp_inband_finish(const TpLink& tp, void* half_base, int64_t bytes) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(tp.counter, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!s_last) return;
  uint4* p = reinterpret_cast<uint4*>(half_base);
  const uint4 e = make_uint4(kTpEmpty2, kTpEmpty2, kTpEmpty2, kTpEmpty2);
  const int64_t n16 = bytes / 16, nthr = blockDim.x;
  int64_t i = threadIdx.x;
  for (; i + 3 * nthr < n16; i += 4 * nthr) {  // four independent stores per thread and round
    p[i] = e;
    p[i + nthr] = e;
    p[i + 2 * nthr] = e;
    p[i + 3 * nthr] = e;
  }
  for (; i < n16; i += nthr) p[i] = e;
  if (threadIdx.x == 0) *tp.counter = 0;
}

__device__ __forceinline__ void ring_flush(Ring& r, PipeCtl& c, int lane) {
  pdl_wait();
  if (r.trigger_after_wait) pdl_launch_dependents();
  if (r.tp != nullptr && !r.tp->inband && !tp_link_wait(*r.tp, lane)) {
    // the copies still go out (the consumers' barriers expect them); the result is flagged as not to be trusted
    if (lane == 0) set_status(r.status, SLORA_STATUS_TIMEOUT);
  }
  PipeCtl::Prod& pp = c.prod[r.role];
  for (int i = 0; i < r.npend; ++i) {
    const uint32_t slot = (r.g - r.npend + i) % kSlots;
    if (pp.pend_bytes[i][lane] != 0) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       pp.pend_dst[i][lane]),
                   "l"(pp.pend_src[i][lane]), "r"(pp.pend_bytes[i][lane]), "r"(smem_u32(&c.full[slot]))
                   : "memory");
    }
  }
  r.npend = 0;
  r.pre = false;
}

// Reserve `sz` bytes (a multiple of 128) and a descriptor for stage r.g; returns the byte offset, or 0xffffffff when
// a wait ran out.  Before the grid-dependency wait no stage has been released yet, so running out of room there
// ends the prologue (ring_flush) instead of waiting.
__device__ __forceinline__ uint32_t ring_alloc(Ring& r, PipeCtl& c, uint32_t sz, int lane) {
  for (;;) {
    uint32_t cand = 0;
    bool ok;
    if (r.tail == r.g) {
      r.head = 0;
      ok = true;
    } else {
      const uint32_t t = c.prod[r.role].off[r.tail % kSlots];
      if (r.head > t) {
        if (r.head + sz <= r.cap) {
          cand = r.head;
          ok = true;
        } else {
          cand = 0;
          ok = sz <= t;
        }
      } else {
        cand = r.head;
        ok = r.head + sz <= t && r.head != t;
      }
    }
    if (ok && r.g - r.tail < kSlots && !(r.pre && r.npend == kPendSlots)) return cand;
    if (r.pre) {
      ring_flush(r, c, lane);
      continue;
    }
    if (!mbar_wait_timed(&c.empty[r.tail % kSlots], (r.tail / kSlots) & 1)) {
      r.dead = true;
      return 0xffffffffu;
    }
    ++r.tail;
  }
}

// One bulk instruction for the whole stage: lane `lane` carries (dst, src, bytes) or bytes == 0.  Activation copies
// (is_act) issued before the grid-dependency wait are stashed instead.
__device__ __forceinline__ void ring_issue(Ring& r, PipeCtl& c, uint32_t slot, uint32_t dst, const void* src,
                                           uint32_t bytes, bool is_act, int lane) {
  if (static_cast<int>(r.g % kProducerWarps) != r.role) bytes = 0;  // the other producer's stage
  if (r.pre) {
    PipeCtl::Prod& pp = c.prod[r.role];
    pp.pend_bytes[r.npend][lane] = is_act ? bytes : 0;
    pp.pend_dst[r.npend][lane] = dst;
    pp.pend_src[r.npend][lane] = reinterpret_cast<uint64_t>(src);
    if (is_act) bytes = 0;
  }
  if (bytes != 0) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(smem_u32(&c.full[slot]))
                 : "memory");
  }
  if (r.pre) ++r.npend;
  ++r.g;
}

// Finish: flush a prologue that never ended, then post the end marker.
__device__ __forceinline__ void ring_finish(Ring& r, PipeCtl& c, int32_t* status, int lane) {
  if (r.pre) ring_flush(r, c, lane);
  if (!r.dead) ring_alloc(r, c, 0, lane);
  if (r.dead) {
    if (lane == 0) set_status(status, SLORA_STATUS_TIMEOUT);
    return;
  }
  const uint32_t slot = r.g % kSlots;
  if (lane == 0 && static_cast<int>(r.g % kProducerWarps) == r.role) {
    c.meta[slot][0] = FLAG_END;
    mbar_arrive(&c.full[slot]);
  }
}

__device__ __forceinline__ void pipe_init(PipeCtl& c, int tid) {
  if (tid == 0) {
    c.tp_gave_up = 0;
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&c.full[s], 1);
      mbar_init(&c.empty[s], kConsumerWarps);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
}

template <typename P>
__device__ __forceinline__ P pick3(P const (&arr)[3], int p) {
  return p == 0 ? arr[0] : (p == 1 ? arr[1] : arr[2]);
}

__device__ __forceinline__ uint32_t round128(uint32_t v) { return (v + 127u) & ~127u; }

// ------------------------------------------------------------------------------------------------------------
// Which items does a launch have?  A tile yields a number of items that depends on its adapter's rank (row blocks
// of the shrink, B chunks of the expand).  Enumerating a fixed number of slots per tile, sized for the widest rank,
// and skipping the empty ones leaves the CTAs (item i belongs to CTA i mod gridDim.x) with unequal shares as soon
// as ranks differ - the empty slots recur with the period of the slot grid.  With a plan the items are therefore
// counted exactly: in closed form when every tile has the same rank (the plan's header says so), else through a
// per-tile running count that the CTA builds in shared memory from the tile records (all threads fetch the
// records, the producer warp scans the counts; before the grid-dependency wait: the plan is complete by then).  Without a plan, or with more tiles or items than the
// control block holds, the padded enumeration stays.  The exact count costs the start of a launch a few hundred
// nanoseconds (its arithmetic sits between the header and the first tile record), which a launch of ten
// microseconds over same-rank adapters does not earn back: the kernels are therefore built both ways (EXACT) and
// the caller, who can ask the plan what it holds (slora_plan_info), picks with SLORA_FLAG_EXACT_ITEMS.
// ------------------------------------------------------------------------------------------------------------
struct ItemMap {
  int mode = 0;      // 0 padded slots, 1 same count for every tile, 2 running count in PipeCtl::item_end
  int per_tile = 0;  // modes 0 and 1
  int uniform = 0;   // mode 1: the slot rows of every tile
  int n_tiles = 0;
  int64_t n_items = 0;
};

// Does this launch count its items per tile (ranks differ, or big groups go elsewhere), and over how many tiles?
__device__ __forceinline__ bool needs_item_counts(const TileSrc& src, int& n_tiles, int& uniform) {
  // the three header words in one go: their loads are on the launch's critical path
  const int32_t* hdr = src.plan;
  const int nt = hdr[PH_NTILES], uni = hdr[PH_UNIFORM], nbig = hdr[PH_NBIG];
  n_tiles = min(nt, src.slots);
  uniform = uni;
  const bool some_elsewhere = src.seg_split > 0 && nbig > 0;  // big groups the tensor-core launch serves
  return !(uni > 0 && !some_elsewhere);
}

// All threads of the CTA: items of every tile into PipeCtl::item_end (one tile record per thread and round, so the
// loads overlap); the caller follows with __syncthreads().
template <typename F>
__device__ __forceinline__ void fill_item_counts(const TileSrc& src, const Tables& tb, PipeCtl& c, int tid,
                                                 F items_of_rank) {
  if (src.mode != MODE_PLAN) return;
  int n_tiles, uniform;
  if (!needs_item_counts(src, n_tiles, uniform) || n_tiles > kCompactTiles) return;
  for (int tile = tid; tile < n_tiles; tile += kPipeThreads) {
    const int4* rec = reinterpret_cast<const int4*>(src.plan + PH_WORDS + kTileWords * tile);
    const int4 r0 = rec[0];
    const int n = r0.z, r = r0.w;
    bool elsewhere = false;
    if (src.seg_split > 0) elsewhere = rec[1].y != 0 && r > 0 && tb.pool_stride % r == 0 && r <= src.mma_max_rows;
    const int cnt = (n > 0 && r > 0 && !elsewhere) ? items_of_rank(r, n) : 0;
    c.item_end[tile] = static_cast<uint16_t>(min(cnt, 0xffff));
  }
}

// Producer warp, after fill_item_counts and the barrier: the launch's item map; with mixed ranks the counts in
// item_end become running counts (each lane sums a contiguous run, the warp scans the lane sums).
template <typename F>
__device__ __forceinline__ ItemMap build_item_map(const TileSrc& src, int padded_per_tile, PipeCtl& c, int lane,
                                                  F items_of_rank) {
  ItemMap m;
  m.per_tile = padded_per_tile;
  if (src.mode != MODE_PLAN) {
    m.n_tiles = src.slots;
    m.n_items = static_cast<int64_t>(m.n_tiles) * padded_per_tile;
    return m;
  }
  int uniform;
  const bool counted = needs_item_counts(src, m.n_tiles, uniform);
  m.n_items = static_cast<int64_t>(m.n_tiles) * padded_per_tile;
  if (!counted) {
    m.mode = 1;
    m.uniform = uniform;
    m.per_tile = items_of_rank(uniform, kTileTokens);
    m.n_items = static_cast<int64_t>(m.n_tiles) * m.per_tile;
    return m;
  }
  if (m.n_tiles > kCompactTiles) return m;
  const int per = (m.n_tiles + 31) / 32;
  const int lo = min(lane * per, m.n_tiles), hi = min(lo + per, m.n_tiles);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += c.item_end[i];
  int incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(FULL_MASK, incl, d);
    if (lane >= d) incl += v;
  }
  const int total = __shfl_sync(FULL_MASK, incl, 31);
  if (total > 0xffff) return m;  // too many items for 16-bit counts (same decision in every lane)
  int run = incl - sum;
  for (int i = lo; i < hi; ++i) {
    run += c.item_end[i];
    c.item_end[i] = static_cast<uint16_t>(run);
  }
  __syncwarp();
  m.mode = 2;
  m.n_items = total;
  return m;
}

// The padded enumeration alone.  Nothing is read from the plan here: the first batch of items is bounded by the tile
// slots the workspace has (tile_lookup tells which of them hold tiles), so that its loads do not queue behind a
// load of the tile count; later batches use the count (padded_item_count), which has arrived by then.
__device__ __forceinline__ ItemMap padded_item_map(const TileSrc& src, int padded_per_tile) {
  ItemMap m;
  m.per_tile = padded_per_tile;
  m.n_tiles = src.slots;
  m.n_items = static_cast<int64_t>(m.n_tiles) * padded_per_tile;
  return m;
}
__device__ __forceinline__ int64_t padded_item_count(const TileSrc& src, int padded_per_tile) {
  return static_cast<int64_t>(tile_count(src)) * padded_per_tile;
}

// Item q -> its tile and its index among that tile's items.
__device__ __forceinline__ void item_to_tile(const ItemMap& m, const PipeCtl& c, int64_t q, int& tile, int& local) {
  if (m.mode != 2) {
    tile = static_cast<int>(q / m.per_tile);
    local = static_cast<int>(q - static_cast<int64_t>(tile) * m.per_tile);
    return;
  }
  int lo = 0, hi = m.n_tiles - 1;  // first tile whose running count exceeds q
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(c.item_end[mid]) > q) {
      hi = mid;
    } else {
      lo = mid + 1;
    }
  }
  tile = lo;
  local = static_cast<int>(q) - (lo > 0 ? c.item_end[lo - 1] : 0);
}

// ------------------------------------------------------------------------------------------------------------
// shrink
// stage meta: [0] flags [1] nrows [2] n [3] j0 [4] projection [5] klen [6] ring offset, [8..15] token ids
// stage bytes: nrows chunks of klen elements (adapter rows), then n chunks of klen elements (token rows)
// ------------------------------------------------------------------------------------------------------------
// Row blocks a tile of rr slot rows has per projection (blocks of kWideRows rows when `wide`, else kMaxRows; rows
// beyond the delta buffers' width are not enumerated), and its items.
__device__ __forceinline__ int shrink_rows_of(const ShrinkArgs& a, int rr) {
  return min(rr * a.rank_mult, a.max_rb * kMaxRows);
}
__device__ __forceinline__ int shrink_blocks_of(const ShrinkArgs& a, int rr, bool wide) {
  const int per = wide ? kWideRows : kMaxRows;
  return (shrink_rows_of(a, rr) + per - 1) / per;
}
// With per-tile counts (ranks differ) a tile of few tokens takes its rows eight at a time: its token rows are then
// staged once per eight adapter rows instead of once per four.
__device__ __forceinline__ int shrink_items_of(const ShrinkArgs& a, int rr, int n) {
  return a.nproj * shrink_blocks_of(a, rr, n <= kWideTokens);
}

template <typename T, bool EXACT>
__device__ __forceinline__ void shrink_producer(const ShrinkArgs& a, unsigned char* ring_mem, PipeCtl& c, int lane,
                                                int role) {
  const int h_in = a.h_in;
  const int64_t S = a.tb.pool_stride;
  const T* w = reinterpret_cast<const T*>(a.w);
  const T* x = reinterpret_cast<const T*>(a.x);
  const int64_t G = gridDim.x;
  const uint32_t ring_base = smem_u32(ring_mem);
  PipeCtl::Prod& pp = c.prod[role];
  Ring r;
  r.role = role;
  r.trigger_after_wait = a.tp.enabled && a.tp.inband >= 2;
  constexpr int RMAX = EXACT ? kWideRows : kMaxRows;  // rows of the widest item = lane of the first token row
  const ItemMap map = EXACT ? build_item_map(a.src, a.nproj * a.max_rb, c, lane,
                                             [&](int rr, int) { return a.nproj * shrink_blocks_of(a, rr, false); })
                            : padded_item_map(a.src, a.nproj * a.max_rb);
  const int mode = EXACT ? map.mode : 0;
  int64_t n_items = map.n_items;
  const int rows_per_pool_row = static_cast<int>(S / h_in);  // the pipelined shrink is given S % h_in == 0

  for (int64_t batch0 = blockIdx.x; batch0 < n_items && !r.dead; batch0 += 32 * G) {
    // ---- 32 items resolved in parallel, one per lane; d_i[lane] = {valid, n, nrows, j0, p, -, -, -, tok[8]} ----
    const int64_t item = batch0 + lane * G;
    int valid = 0;
    if (item < n_items) {
      int tile, rem;
      item_to_tile(map, c, item, tile, rem);
      // projection and row block: known before the tile record arrives unless ranks are mixed
      int nb = mode == 0 ? a.max_rb : shrink_blocks_of(a, map.uniform, false);
      // resolved tiles: where projection and row block follow from the item index alone, the pool rows of the
      // item are fetched now, together with the header and the record that will say whether they count
      int spec_row[kMaxRows];
      bool spec = false;
      if (a.src.mode == MODE_PLAN && a.src.xoff > 0 && mode != 2) {
        const int p_s = min(rem / nb, a.nproj - 1), rb_s = rem - (rem / nb) * nb;
        const int32_t* xt = a.src.plan + a.src.xoff + static_cast<int64_t>(tile) * (kXtHead + 4 * a.src.xrcap);
        const int qk_s = pick3(a.qkvo, p_s);
#pragma unroll
        for (int j = 0; j < kMaxRows; ++j) {
          const int pr = (rb_s * kMaxRows + j) / rows_per_pool_row;
          spec_row[j] = xt[kXtHead + qk_s * a.src.xrcap + min(pr, a.src.xrcap - 1)];
        }
        spec = true;
      }
      TileInfo t;
      if (lookup_tile(a.src, a.tb, tile, t, a.status)) {
        const bool wide = mode == 2 && t.n <= kWideTokens;
        if (mode == 2) nb = shrink_blocks_of(a, t.r, wide);
        const int per = wide ? kWideRows : kMaxRows;
        const int p = rem / nb, rb = rem - p * nb;
        const int j0 = rb * per;
        const int rows_total = shrink_rows_of(a, t.r);  // A rows of the projection (rows may be shorter than a pool row)
        if (p < a.nproj && j0 < rows_total) {
          const int nrows = min(per, rows_total - j0);
          const int qk = pick3(a.qkvo, p);
          bool ok = true;
#pragma unroll
          for (int j = 0; j < RMAX; ++j) {
            if (j < nrows) {
              const int64_t f = static_cast<int64_t>(j0 + j) * h_in;
              const int64_t pr = f / S, col = f - pr * S;
              int64_t e = -1;
              if (pr < t.r) e = (spec && t.xok && j < kMaxRows) ? spec_row[j < kMaxRows ? j : 0] : tile_loc(t, a.tb, qk, pr);
              if (e < 0 || e >= a.tb.pool_rows) ok = false;
              pp.d_l[lane][j] = e * S + col;
            }
          }
          if (ok) {
#pragma unroll
            for (int i = 0; i < kTileTokens; ++i) pp.d_i[lane][8 + i] = i < t.n ? tile_token(t, i) : 0;
            pp.d_i[lane][1] = t.n;
            pp.d_i[lane][2] = nrows;
            pp.d_i[lane][3] = j0;
            pp.d_i[lane][4] = p;
            pp.d_i[lane][5] = t.r;
            valid = 1;
          } else {
            set_status(a.status, SLORA_STATUS_BAD_TABLE);
          }
        }
      }
    }
    const uint32_t valid_mask = __ballot_sync(FULL_MASK, valid != 0);
    __syncwarp();

    // ---- feed the ring, item by item (lane j < RMAX carries adapter row j, lane RMAX + i carries token i) ----
    for (uint32_t left = valid_mask; left != 0 && !r.dead; left &= left - 1) {
      const int k = __ffs(left) - 1;
      const int* di = pp.d_i[k];
      const int n = di[1], nrows = di[2];
      const bool is_w = lane < nrows;
      const bool is_x = lane >= RMAX && lane < RMAX + n;
      const int mytok = (lane >= RMAX && lane < RMAX + kTileTokens) ? di[8 + lane - RMAX] : 0;
      const T* src0 = is_w ? w + pp.d_l[k][lane & (RMAX - 1)] : x + static_cast<int64_t>(mytok) * a.x_stride;
      const int myslot = is_w ? lane : nrows + (lane - RMAX);  // position of this lane's chunk in the stage
      const int m_j0 = di[3], m_p = di[4], m_rows = di[5];
      // cut the item into K-chunks that are multiples of 2048 elements (so the element -> consumer lane mapping, and
      // with it the summation order, does not depend on how many tokens share the tile) and, where that allows,
      // no larger than kMaxStageBytes
      const int fit = kMaxStageBytes / ((nrows + n) * static_cast<int>(sizeof(T))) / 2048 * 2048;
      const int kc_elems = fit < 2048 ? 2048 : fit;
      for (int k0 = 0; k0 < h_in; k0 += kc_elems) {
        const int klen = min(kc_elems, h_in - k0);
        const uint32_t bytes = static_cast<uint32_t>(klen) * sizeof(T);
        const uint32_t sz = round128(static_cast<uint32_t>(nrows + n) * bytes);
        const uint32_t off = ring_alloc(r, c, sz, lane);
        if (r.dead) break;
        const uint32_t slot = r.g % kSlots;
        const bool mine = static_cast<int>(r.g % kProducerWarps) == role;
        r.head = off + sz;
        if (lane == 0) pp.off[slot] = off;
        if (!mine) {
          __syncwarp();
          ring_issue(r, c, slot, 0, nullptr, 0u, false, lane);
          continue;
        }
        if (lane == 0) {  // the stage record in two 16-byte stores; [7] = slot rows of the adapter
          int4* mrec = reinterpret_cast<int4*>(c.meta[slot]);
          mrec[0] = make_int4((k0 == 0 ? FLAG_FIRST : 0) | (k0 + klen >= h_in ? FLAG_LAST : 0), nrows, n, m_j0);
          mrec[1] = make_int4(m_p, klen, static_cast<int>(off), m_rows);
        } else if (lane >= RMAX && lane < RMAX + kTileTokens) {
          c.meta[slot][8 + lane - RMAX] = mytok;
        }
        __syncwarp();  // the arrive below publishes every lane's part of the stage record
        if (lane == 0) mbar_expect_tx(&c.full[slot], static_cast<uint32_t>(nrows + n) * bytes);
        ring_issue(r, c, slot, ring_base + off + static_cast<uint32_t>(myslot) * bytes, src0 + k0,
                   (is_w || is_x) ? bytes : 0u, is_x, lane);
      }
    }
    __syncwarp();
    if (!EXACT && a.src.mode == MODE_PLAN) n_items = padded_item_count(a.src, a.nproj * a.max_rb);
  }
  ring_finish(r, c, a.status, lane);
}

// Warp-level part of the per-item reduction: V = 4 * NT partial sums per lane (row-major [row][token]) are summed
// across the warp and handed to the cross-warp buffer; lane l ends up with the total of index l >> (5 - log2 V).
template <int NT>
__device__ __forceinline__ void shrink_warp_reduce(const float (&acc)[kMaxRows][kTileTokens], float* red_row, int lane) {
  constexpr int V = kMaxRows * NT;
  float v[V];
#pragma unroll
  for (int j = 0; j < kMaxRows; ++j) {
#pragma unroll
    for (int i = 0; i < NT; ++i) v[j * NT + i] = acc[j][i];
  }
  const float tot = warp_reduce_scatter<V>(v, lane);
  constexpr int SH = V == 32 ? 0 : (V == 16 ? 1 : (V == 8 ? 2 : 3));
  if ((lane & ((1 << SH) - 1)) == 0) red_row[lane >> SH] = tot;
}

// Multiply-accumulate part of a shrink stage for a tile of at most NT tokens, free of data-dependent branches (each
// branch costs the lone warp of a scheduler ~10-20 cycles of resolve latency): rows and tokens beyond the real counts
// are clamped to the last real one, so their accumulators hold duplicates that are never written out.
template <typename T, int NT>
__device__ __forceinline__ void shrink_accumulate(float (&acc)[kMaxRows][kTileTokens], const T* st, int nrows, int n,
                                                  int klen, int cw, int lane) {
  const T* xs = st + nrows * klen;
  const T* wrow[kMaxRows];
#pragma unroll
  for (int j = 0; j < kMaxRows; ++j) wrow[j] = st + min(j, nrows - 1) * klen;
  const T* xrow[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) xrow[i] = xs + min(i, n - 1) * klen;
#pragma unroll 1
  for (int k = cw * 256 + lane * 8; k < klen; k += kConsumerWarps * 256) {
    uint4 wv[kMaxRows];
#pragma unroll
    for (int j = 0; j < kMaxRows; ++j) wv[j] = *reinterpret_cast<const uint4*>(wrow[j] + k);
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xrow[i] + k);
#pragma unroll
      for (int j = 0; j < kMaxRows; ++j) dot8<T>(acc[j][i], wv[j], xv);
    }
  }
}

// The same two steps for an item of kWideRows rows and at most kWideTokens tokens (NT in 1, 2, 4): the 32
// accumulators are the same registers, indexed [row * NT + token].
#define SLORA_ACC(idx) acc[(idx) >> 3][(idx) & 7]
template <typename T, int NT>
__device__ __forceinline__ void shrink_accumulate_wide(float (&acc)[kMaxRows][kTileTokens], const T* st, int nrows,
                                                       int n, int klen, int cw, int lane) {
  const T* xs = st + nrows * klen;
#pragma unroll 1
  for (int k = cw * 256 + lane * 8; k < klen; k += kConsumerWarps * 256) {
    uint4 xv[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) xv[i] = *reinterpret_cast<const uint4*>(xs + min(i, n - 1) * klen + k);
#pragma unroll
    for (int j = 0; j < kWideRows; ++j) {
      const uint4 wv = *reinterpret_cast<const uint4*>(st + min(j, nrows - 1) * klen + k);
#pragma unroll
      for (int i = 0; i < NT; ++i) dot8<T>(SLORA_ACC(j * NT + i), wv, xv[i]);
    }
  }
}
template <int NT>
__device__ __forceinline__ void shrink_warp_reduce_wide(const float (&acc)[kMaxRows][kTileTokens], float* red_row,
                                                        int lane) {
  constexpr int V = kWideRows * NT;
  float v[V];
#pragma unroll
  for (int q = 0; q < V; ++q) v[q] = SLORA_ACC(q);
  const float tot = warp_reduce_scatter<V>(v, lane);
  constexpr int SH = V == 32 ? 0 : (V == 16 ? 1 : 2);
  if ((lane & ((1 << SH) - 1)) == 0) red_row[lane >> SH] = tot;
}
#undef SLORA_ACC

// Consumer warp cw owns the K-slice [cw*256, +256) of every chunk: one 16-byte vector per lane per row / token, so a
// stage is straight-line code with 4 * n independent FMA chains.  At the item's last chunk the warps' partial sums
// meet in shared memory; the warp that arrives last (an atomic counter, no waiting) adds them in a fixed order and
// writes delta.  A reduction buffer is reused only kSlots items later, which the ring guarantees to be after the
// last warp released the stage it was summing in.
template <typename T, bool EXACT>
__device__ __forceinline__ void shrink_consumer(const ShrinkArgs& a, const unsigned char* ring_mem, PipeCtl& c,
                                                ShrinkRed& red, int lane, int cw) {
  pdl_wait();
  int tp_slot = a.tp.half;  // which part of every rank's delta buffer this exchange writes
  if (a.tp.enabled && a.tp.inband == 3) {
    // rotating thirds (see TpLink::inband): the exchange's number picks the third; this CTA's share of the third
    // the PREVIOUS exchange used - whose expand on this GPU is complete: it is what the wait above waited for - goes
    // back to the empty pattern; one thread tells this exchange's expand its number
    const int e = *reinterpret_cast<volatile const int32_t*>(a.tp.seq_state);
    tp_slot = e % 3;
    const int64_t third = 3 * a.tp.full_tokens * static_cast<int64_t>(a.tp.n_parts) * a.delta_width;  // elements
    uint4* prev = reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.tp.full[a.tp.my_part]) + ((e + 2) % 3) * third);
    const int64_t n16 = third * static_cast<int64_t>(sizeof(T)) / 16;
    const uint4 ev = make_uint4(kTpEmpty2, kTpEmpty2, kTpEmpty2, kTpEmpty2);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * (kConsumerWarps * 32) + cw * 32 + lane; i < n16;
         i += static_cast<int64_t>(gridDim.x) * (kConsumerWarps * 32))
      prev[i] = ev;
    if (blockIdx.x == 0 && cw == 0 && lane == 0) {
      a.tp.seq_state[1] = e;
      __threadfence();  // before this thread lets dependents launch
    }
    __syncwarp();
  }
  if (a.tp.enabled && a.tp.inband >= 2) pdl_launch_dependents();
  float acc[kMaxRows][kTileTokens];
#pragma unroll
  for (int j = 0; j < kMaxRows; ++j) {
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) acc[j][i] = 0.f;
  }
  uint32_t item_seq = 0;
  for (uint32_t g = 0;; ++g) {
    const uint32_t slot = g % kSlots;
    if (!mbar_wait_timed(&c.full[slot], (g / kSlots) & 1)) {
      if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
      return;
    }
    const int* m = c.meta[slot];
    const int flags = m[0];
    if (flags & FLAG_END) return;
    const int nrows = m[1], n = m[2], klen = m[5];
    if (flags & FLAG_FIRST) {
#pragma unroll
      for (int j = 0; j < kMaxRows; ++j) {
#pragma unroll
        for (int i = 0; i < kTileTokens; ++i) acc[j][i] = 0.f;
      }
    }
    const T* st = reinterpret_cast<const T*>(ring_mem + m[6]);
    const bool wide = EXACT && nrows > kMaxRows;  // an item of up to kWideRows rows (the tile has <= kWideTokens tokens)
    if (wide) {
      if (n <= 1) {
        shrink_accumulate_wide<T, 1>(acc, st, nrows, n, klen, cw, lane);
      } else if (n <= 2) {
        shrink_accumulate_wide<T, 2>(acc, st, nrows, n, klen, cw, lane);
      } else {
        shrink_accumulate_wide<T, 4>(acc, st, nrows, n, klen, cw, lane);
      }
    } else if (n <= 1) {
      shrink_accumulate<T, 1>(acc, st, nrows, n, klen, cw, lane);
    } else if (n <= 2) {
      shrink_accumulate<T, 2>(acc, st, nrows, n, klen, cw, lane);
    } else if (n <= 4) {
      shrink_accumulate<T, 4>(acc, st, nrows, n, klen, cw, lane);
    } else {
      shrink_accumulate<T, 8>(acc, st, nrows, n, klen, cw, lane);
    }
    if (flags & FLAG_LAST) {
      const uint32_t buf = item_seq % kSlots;
      ++item_seq;
      float* red_row = red.sum[buf][cw];
      int nt;  // tokens rounded up to a power of two
      if (wide) {
        if (n <= 1) {
          shrink_warp_reduce_wide<1>(acc, red_row, lane);
          nt = 1;
        } else if (n <= 2) {
          shrink_warp_reduce_wide<2>(acc, red_row, lane);
          nt = 2;
        } else {
          shrink_warp_reduce_wide<4>(acc, red_row, lane);
          nt = 4;
        }
      } else if (n <= 1) {
        shrink_warp_reduce<1>(acc, red_row, lane);
        nt = 1;
      } else if (n <= 2) {
        shrink_warp_reduce<2>(acc, red_row, lane);
        nt = 2;
      } else if (n <= 4) {
        shrink_warp_reduce<4>(acc, red_row, lane);
        nt = 4;
      } else {
        shrink_warp_reduce<8>(acc, red_row, lane);
        nt = 8;
      }
      __syncwarp();
      int old = 0;
      if (lane == 0) {
        __threadfence_block();
        old = atomicAdd(&red.cnt[buf], 1);
      }
      old = __shfl_sync(FULL_MASK, old, 0);
      if (old == kConsumerWarps - 1) {
        __threadfence_block();
        const int j = lane / nt, i = lane - j * nt;  // red_row index = row * nt + token
        if (lane < (wide ? kWideRows : kMaxRows) * nt) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) sum += red.sum[buf][w][lane];
          if (j < nrows && i < n && m[3] + j < a.delta_width) {
            if (a.tp.enabled) {
              // tensor parallelism: this rank's rows go straight into every rank's delta buffer (NVLink stores)
              const int64_t R = static_cast<int64_t>(a.tp.n_parts) * a.delta_width;
              const int64_t at = ((static_cast<int64_t>(tp_slot) * 3 + m[4]) * a.tp.full_tokens + m[8 + i]) * R +
                                 static_cast<int64_t>(a.tp.my_part) * m[7] + m[3] + j;
              const T v = from_f32<T>(sum);
              for (int g = 0; g < a.tp.n_parts; ++g) reinterpret_cast<T*>(a.tp.full[g])[at] = v;
            } else {
              T* d = reinterpret_cast<T*>(pick3(a.delta, m[4]));
              d[static_cast<int64_t>(m[8 + i]) * a.delta_stride + m[3] + j] = from_f32<T>(sum);
            }
          }
        }
        if (lane == 0) red.cnt[buf] = 0;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
}

// A segment call sends its long segments to the tensor-core kernels and launches these kernels beside them for the
// short ones.  When there are none (a pure prefill batch) the launch has nothing to do: every CTA finds that out from
// the segment table with one round of loads per table (a thread per segment) and leaves before it sets up its ring,
// instead of resolving every tile slot of every segment first.  A segment whose table entries look wrong counts as
// this launch's, whose normal path reports it.
__device__ __forceinline__ bool segments_all_elsewhere(const TileSrc& s, const Tables& tb) {
  if (s.mode != MODE_SEGMENT || s.seg_split <= 0) return false;
  bool mine = false;
  for (int i = threadIdx.x; i < s.n_seg; i += blockDim.x) {
    const int64_t len = s.seg_len[i];
    if (len <= 0) continue;
    const int64_t ad = s.ids[i];
    if (len < s.seg_split || ad < 0 || ad >= tb.n_adapters) {
      mine = true;
      continue;
    }
    const int64_t r4 = tb.ranks4[ad], st = tb.start[ad], r = r4 >> 2;
    if (r4 < 0 || st < 0 || st + r4 > tb.loc_len ||
        !(r >= 8 && r <= 128 && r % 8 == 0 && tb.pool_stride % r == 0 && r <= s.mma_max_rows))
      mine = true;
  }
  return __syncthreads_or(mine) == 0;
}

template <typename T, bool EXACT>
__global__ void __launch_bounds__(kPipeThreads, kPipeCtasPerSm) lora_shrink_pipe_kernel(const ShrinkArgs a) {
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(16) PipeCtl ctl;
  __shared__ __align__(16) ShrinkRed red;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (segments_all_elsewhere(a.src, a.tb)) return;
  if (tid < kSlots) red.cnt[tid] = 0;
  pipe_init(ctl, tid);
  // (a shrink whose expand starts early lets its dependents launch only after its own grid-dependency wait, thread
  // by thread: see TpLink::inband)
  if (!(a.tp.enabled && a.tp.inband >= 2)) pdl_launch_dependents();
  if (EXACT) {
    fill_item_counts(a.src, a.tb, ctl, tid, [&](int rr, int n) { return shrink_items_of(a, rr, n); });
    __syncthreads();
  }
  if (warp < kProducerWarps) {
    shrink_producer<T, EXACT>(a, ring_mem, ctl, lane, warp);
  } else {
    shrink_consumer<T, EXACT>(a, ring_mem, ctl, red, lane, warp - kProducerWarps);
  }
  if (a.tp.enabled && !a.tp.inband) tp_link_finish(a.tp, true);
}

// ------------------------------------------------------------------------------------------------------------
// expand
// stage meta: [0] flags [1] n [2] r [3] projection [4] clen [5] first output [6] scale bits [7] ring offset,
//             [8..15] token ids
// stage bytes: B chunk (clen elements), then n y segments of clen / r elements, then n delta rows of r elements
// ------------------------------------------------------------------------------------------------------------
// The expand takes ranks 8..128 in powers of two that the delta buffers hold; B chunks of projection p for rank rk;
// items of a tile of rr slot rows.
__device__ __forceinline__ bool expand_rank_ok(const ExpandArgs& a, int rk) {
  return (rk == 8 || rk == 16 || rk == 32 || rk == 64 || rk == 128) && rk <= a.max_rank;
}
__device__ __forceinline__ int expand_chunks_of(const ExpandArgs& a, int p, int rk) {
  const int64_t flat = static_cast<int64_t>(pick3(a.h_out, p)) * rk;
  return static_cast<int>(min(static_cast<int64_t>(a.chunk_begin[p + 1] - a.chunk_begin[p]),
                              (flat + kPipeChunk - 1) / kPipeChunk));
}
__device__ __forceinline__ int expand_items_of(const ExpandArgs& a, int rr) {
  const int rk = rr * a.rank_mult;
  if (!expand_rank_ok(a, rk)) return 1;  // one item, which reports the rank
  int n = 0;
  for (int p = 0; p < a.nproj; ++p) n += expand_chunks_of(a, p, rk);
  return n;
}

template <typename T, bool EXACT>
__device__ __forceinline__ void expand_producer(const ExpandArgs& a, unsigned char* ring_mem, PipeCtl& c, int lane,
                                                int role) {
  const int total_chunks = a.chunk_begin[a.nproj];
  const int64_t S = a.tb.pool_stride;
  const T* w = reinterpret_cast<const T*>(a.w);
  const int64_t G = gridDim.x;
  const uint32_t ring_base = smem_u32(ring_mem);
  PipeCtl::Prod& pp = c.prod[role];
  Ring r;
  r.role = role;
  r.cap = EXACT ? kExpandRingBytes : kRingBytes;  // see kExpandRingBytes
  r.tp = a.tp.enabled ? &a.tp : nullptr;
  r.status = a.status;
  if (a.tp.enabled && a.tp.inband >= 2) r.pre = false;  // early start: nothing to wait for (see TpLink::inband)
  int64_t delta_off = 0;  // rotating thirds: elements from the first third to this exchange's
  if (a.tp.enabled && a.tp.inband == 3) {
    const int e = *reinterpret_cast<volatile const int32_t*>(a.tp.seq_state + 1);  // left by this exchange's shrink
    delta_off = (e % 3) * 3 * a.tp.full_tokens * a.delta_stride;
    if (blockIdx.x == 0 && lane == 0) a.tp.seq_state[0] = e + 1;  // the next shrink reads it after its own wait
  }
  auto rank_ok = [&](int rk) { return expand_rank_ok(a, rk); };
  auto chunks_of = [&](int p, int rk) { return expand_chunks_of(a, p, rk); };
  const ItemMap map = EXACT ? build_item_map(a.src, total_chunks, c, lane, [&](int rr, int) { return expand_items_of(a, rr); })
                            : padded_item_map(a.src, total_chunks);
  const int mode = EXACT ? map.mode : 0;
  int64_t n_items = map.n_items;

  for (int64_t batch0 = blockIdx.x; batch0 < n_items && !r.dead; batch0 += 32 * G) {
    // d_i[lane] = {pr0, n, r, p, clen, first output, scale bits, chunk start inside pool row pr0, tok[8]},
    // d_l[lane][j] = pool row of slot row pr0 + j
    const int64_t item = batch0 + lane * G;
    int valid = 0;
    if (item < n_items) {
      int tile, ch;
      item_to_tile(map, c, item, tile, ch);
      // projection and chunk: known before the tile record arrives unless ranks are mixed
      int p = 0;
      auto split = [&](int rk) {
        while (p + 1 < a.nproj && ch >= chunks_of(p, rk)) {
          ch -= chunks_of(p, rk);
          ++p;
        }
      };
      if (mode == 0) {
        while (p + 1 < a.nproj && ch >= a.chunk_begin[p + 1]) ++p;
        ch -= a.chunk_begin[p];
      } else if (mode == 1 && rank_ok(map.uniform * a.rank_mult)) {
        split(map.uniform * a.rank_mult);
      }
      // resolved tiles: where projection and chunk follow from the item index alone, the chunk's pool rows and the
      // adapter's scale are fetched now, together with the header and the record that will say whether they count
      int spec_row[kSpanRows], spec_scale = 0;
      bool spec = false;
      if (a.src.mode == MODE_PLAN && a.src.xoff > 0 && mode != 2) {
        const int32_t* xt = a.src.plan + a.src.xoff + static_cast<int64_t>(tile) * (kXtHead + 4 * a.src.xrcap);
        const int qk_s = pick3(a.qkvo, p);
        const int pr_s = static_cast<int>(static_cast<int64_t>(ch) * kPipeChunk / S);
        spec_scale = xt[8];
#pragma unroll
        for (int j = 0; j < kSpanRows; ++j)
          spec_row[j] = xt[kXtHead + qk_s * a.src.xrcap + min(pr_s + j, a.src.xrcap - 1)];
        spec = true;
      }
      TileInfo t;
      if (lookup_tile(a.src, a.tb, tile, t, a.status)) {
        const int rk = t.r * a.rank_mult;
        if (mode == 2 && rank_ok(rk)) split(rk);
        const int h_out = pick3(a.h_out, p);
        const int64_t flat_total = static_cast<int64_t>(h_out) * rk;
        const int64_t c0 = static_cast<int64_t>(ch) * kPipeChunk;
        if (c0 < flat_total) {
          if (!rank_ok(rk)) {
            set_status(a.status, SLORA_STATUS_BAD_RANK);
          } else {
            const int clen = static_cast<int>(min(static_cast<int64_t>(kPipeChunk), flat_total - c0));
            const int qk = pick3(a.qkvo, p);
            const int64_t pr0 = c0 / S, pr1 = (c0 + clen - 1) / S;
            bool ok = pr1 - pr0 < kSpanRows && pr1 < t.r;
            if (ok) {
#pragma unroll
              for (int j = 0; j < kSpanRows; ++j) {
                if (pr0 + j <= pr1) {
                  const int64_t e = (spec && t.xok) ? spec_row[j] : tile_loc(t, a.tb, qk, pr0 + j);
                  if (e < 0 || e >= a.tb.pool_rows) ok = false;
                  pp.d_l[lane][j] = e;
                }
              }
            }
            if (ok) {
#pragma unroll
              for (int i = 0; i < kTileTokens; ++i) pp.d_i[lane][8 + i] = i < t.n ? tile_token(t, i) : 0;
              pp.d_i[lane][0] = static_cast<int>(pr0);
              pp.d_i[lane][1] = t.n;
              pp.d_i[lane][2] = rk;
              pp.d_i[lane][3] = p;
              pp.d_i[lane][4] = clen;
              pp.d_i[lane][5] = static_cast<int>(c0 / rk);
              {
                // the scale's 16 bits: from the resolved tile when it counts and carries one, else from the table
                T sc;
                if (spec && t.xok && (spec_scale & 0x10000)) {
                  const unsigned short bits = static_cast<unsigned short>(spec_scale & 0xffff);
                  sc = *reinterpret_cast<const T*>(&bits);
                } else {
                  sc = reinterpret_cast<const T*>(a.scales)[t.adapter];
                }
                pp.d_i[lane][6] = __float_as_int(to_f32<T>(sc));
              }
              pp.d_i[lane][7] = static_cast<int>(c0 - pr0 * S);  // chunk start inside its first pool row
              valid = 1;
            } else {
              set_status(a.status, SLORA_STATUS_BAD_TABLE);
            }
          }
        }
      }
    }
    const uint32_t valid_mask = __ballot_sync(FULL_MASK, valid != 0);
    __syncwarp();

    // one copy per lane: 0..15 pieces of the B chunk, 16..23 y segments, 24..31 delta rows.  Everything that does
    // not depend on where the stage lands in the ring is worked out BEFORE the wait for ring space: what follows the
    // wait is on the path from a consumer's release of a stage to the next copy's issue.
    for (uint32_t left = valid_mask; left != 0 && !r.dead; left &= left - 1) {
      const int k = __ffs(left) - 1;
      const int* di = pp.d_i[k];
      const int n = di[1], rk = di[2], p = di[3], clen = di[4], obase = di[5];
      const int nout = clen / rk;
      const uint32_t b_bytes = static_cast<uint32_t>(clen) * sizeof(T);
      const uint32_t y_bytes = static_cast<uint32_t>(nout) * sizeof(T);
      const uint32_t d_bytes = static_cast<uint32_t>(rk) * sizeof(T);
      const uint32_t total = b_bytes + static_cast<uint32_t>(n) * (y_bytes + d_bytes);
      const uint32_t sz = round128(total);
      const int mytok = lane >= 16 ? di[8 + (lane & 7)] : 0;
      uint32_t rel = 0, bytes = 0;  // this lane's copy: offset inside the stage, size
      const T* src = w;
      bool is_act = false;
      if (lane < kMaxPieces) {
        const int poff = lane * a.piece;
        if (poff < clen) {
          const int f = di[7] + poff;  // offset from the start of the chunk's first pool row
          const int pr = f / static_cast<int>(S), col = f - pr * static_cast<int>(S);
          src = w + pp.d_l[k][pr] * S + col;
          rel = static_cast<uint32_t>(poff) * sizeof(T);
          bytes = static_cast<uint32_t>(min(a.piece, clen - poff)) * sizeof(T);
        }
      } else if (lane < 16 + n) {
        src = reinterpret_cast<const T*>(pick3(a.y, p)) + static_cast<int64_t>(mytok) * pick3(a.y_stride, p) + obase;
        rel = b_bytes + static_cast<uint32_t>(lane - 16) * y_bytes;
        bytes = y_bytes;
        is_act = true;
      } else if (lane >= 24 && lane < 24 + n) {
        src = reinterpret_cast<const T*>(pick3(a.delta, p)) + delta_off + static_cast<int64_t>(mytok) * a.delta_stride;
        rel = b_bytes + static_cast<uint32_t>(n) * y_bytes + static_cast<uint32_t>(lane - 24) * d_bytes;
        bytes = d_bytes;
        is_act = true;
      }
      const int m_scale = di[6];
      const uint32_t off = ring_alloc(r, c, sz, lane);
      if (r.dead) break;
      const uint32_t slot = r.g % kSlots;
      const bool mine = static_cast<int>(r.g % kProducerWarps) == role;
      r.head = off + sz;
      if (lane == 0) pp.off[slot] = off;
      if (!mine) {
        __syncwarp();
        ring_issue(r, c, slot, 0, nullptr, 0u, false, lane);
        continue;
      }
      if (lane == 0) {  // the stage record in two 16-byte stores
        int4* mrec = reinterpret_cast<int4*>(c.meta[slot]);
        mrec[0] = make_int4(0, n, rk, p);
        mrec[1] = make_int4(clen, obase, m_scale, static_cast<int>(off));
      } else if (lane >= 16 && lane < 24) {
        c.meta[slot][8 + lane - 16] = mytok;
      }
      __syncwarp();  // the arrive below publishes every lane's part of the stage record
      if (lane == 0) mbar_expect_tx(&c.full[slot], total);
      ring_issue(r, c, slot, ring_base + off + rel, src, bytes, is_act, lane);
    }
    __syncwarp();
    if (!EXACT && a.src.mode == MODE_PLAN) n_items = padded_item_count(a.src, total_chunks);
  }
  ring_finish(r, c, a.status, lane);
}

// Tensor parallelism with in-band signalling: before a warp uses a stage, it looks at the delta values the stage's
// copy brought.  The common case - everything had landed - costs each lane one look at the vectors it is going to
// use (the 16 bytes at its own k offset of each of the n rows) and the warp one vote.  Otherwise the warp settles the
// whole delta block: lane l takes the vectors l, l + 32, ...; one that still holds the empty pattern is fetched again
// from global memory until it has arrived (bounded) and put into the stage.  Every warp does this by itself (the
// warps do not wait for one another; they write the same values), so the arithmetic that follows is the same
// straight loop as without tensor parallelism.
template <typename T>
__device__ __noinline__ void expand_settle_slow(T* ds, const int* m, int r, const T* dglobal, int64_t dglobal_stride,
                                                int32_t* status, volatile int* gave_up, int lane);

template <typename T>
__device__ __forceinline__ void expand_settle_delta(T* ds, const int* m, int r, const T* dglobal, int64_t dglobal_stride,
                                                    int32_t* status, volatile int* gave_up, int lane) {
  const int n = m[1];
  const int kp = (lane & (r / 8 - 1)) * 8;  // r is a power of two (expand_rank_ok)
  bool missing = false;
  for (int tt = 0; tt < n; ++tt) missing |= tp_has_empty(*reinterpret_cast<const uint4*>(ds + tt * r + kp));
  if (__any_sync(FULL_MASK, missing)) expand_settle_slow<T>(ds, m, r, dglobal, dglobal_stride, status, gave_up, lane);
}

// (kept out of line: it runs once in a long while and its polling loop would only bloat the consumers' hot loop)
template <typename T>
__device__ __noinline__ void expand_settle_slow(T* ds, const int* m, int r, const T* dglobal, int64_t dglobal_stride,
                                                int32_t* status, volatile int* gave_up, int lane) {
  const int n = m[1];
  const int vec_per_row = r / 8;
  for (int v = lane; v < n * vec_per_row; v += 32) {
    const int tt = v / vec_per_row, k0 = (v - tt * vec_per_row) * 8;
    uint4 dv = *reinterpret_cast<const uint4*>(ds + tt * r + k0);
    if (tp_has_empty(dv)) {
      if (!tp_poll_delta(dglobal + static_cast<int64_t>(m[8 + tt]) * dglobal_stride + k0, dv, gave_up)) {
        set_status(status, SLORA_STATUS_TIMEOUT);
        dv = make_uint4(0u, 0u, 0u, 0u);
      }
      *reinterpret_cast<uint4*>(ds + tt * r + k0) = dv;
      fence_proxy_async();  // this store before the bulk copy that will reuse the stage's bytes
    }
  }
  __syncwarp();
}

// One consumer warp's part of an expand stage.  LPO = lanes per output = r / 8.  The warp owns flat elements
// [cw*2048, +2048) of the chunk as 8 loads of 256 elements; load m, lane l holds the 8 values of output
// (cw*8 + m)*(32/LPO) + l/LPO for k in [(l % LPO)*8, +8).
template <typename T, int LPO, bool FULL, bool INBAND = false>
__device__ __forceinline__ void expand_stage(const T* bs, const int* m, T* y, int64_t y_stride, int lane, int cw,
                                             const T* dglobal = nullptr, int64_t dglobal_stride = 0,
                                             int32_t* status = nullptr, volatile int* gave_up = nullptr) {
  constexpr int OPL = 32 / LPO;
  constexpr int NV = LPO >= 8 ? 1 : 8 / LPO;
  constexpr int R = LPO * 8;
  constexpr int SPAN = kPipeChunk / kConsumerWarps;  // 2048
  const int n = m[1], clen = m[4], obase = m[5];
  if (cw * SPAN >= clen) return;
  const int nout = clen / R;
  const float scale = __int_as_float(m[6]);
  const T* ys = bs + clen;
  const T* ds = ys + n * nout;
  uint4 bv[8];
#pragma unroll
  for (int mm = 0; mm < 8; ++mm) {
    const int foff = cw * SPAN + mm * 256 + lane * 8;
    bv[mm] = (FULL || foff < clen) ? *reinterpret_cast<const uint4*>(bs + foff) : make_uint4(0u, 0u, 0u, 0u);
  }
  // in-band signalling: have this stage's delta values all arrived?  (after the B loads have been issued, so that the
  // look costs no latency of its own)
  if (INBAND) expand_settle_delta<T>(const_cast<T*>(ds), m, R, dglobal, dglobal_stride, status, gave_up, lane);
  const int kp = (lane & (LPO - 1)) * 8;
  const int g = lane / LPO;
  const int m_base = expand_m_base<LPO>(lane);
  const bool writer = (LPO < 16) || ((lane & 8) == 0);
  int o_loc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o_loc[i] = (cw * 8 + m_base + i) * OPL + g;  // output index inside the chunk

  for (int tt = 0; tt < n; ++tt) {
    const uint4 dv = *reinterpret_cast<const uint4*>(ds + tt * R + kp);
    float yv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      yv[i] = (FULL || (writer && o_loc[i] < nout)) ? to_f32<T>(ys[tt * nout + o_loc[i]]) : 0.f;
    }
    float v[8];
#pragma unroll
    for (int mm = 0; mm < 8; ++mm) {
      v[mm] = 0.f;
      dot8<T>(v[mm], bv[mm], dv);
    }
    expand_butterfly<LPO>(v, lane);
    T* yrow = y + static_cast<int64_t>(m[8 + tt]) * y_stride + obase;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (writer && (FULL || o_loc[i] < nout)) yrow[o_loc[i]] = from_f32<T>(fmaf(scale, v[i], yv[i]));
    }
  }
}

template <typename T, bool INBAND>
__device__ __forceinline__ void expand_consumer(const ExpandArgs& a, const unsigned char* ring_mem, PipeCtl& c,
                                                int lane, int cw) {
  if (!(a.tp.enabled && a.tp.inband >= 2)) pdl_wait();
  int64_t delta_off = 0;
  if (INBAND && a.tp.inband == 3)
    delta_off = (*reinterpret_cast<volatile const int32_t*>(a.tp.seq_state + 1) % 3) * 3 * a.tp.full_tokens *
                a.delta_stride;
  for (uint32_t g = 0;; ++g) {
    const uint32_t slot = g % kSlots;
    if (!mbar_wait_timed(&c.full[slot], (g / kSlots) & 1)) {
      if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
      return;
    }
    const int* m = c.meta[slot];
    if (m[0] & FLAG_END) return;
    const T* bs = reinterpret_cast<const T*>(ring_mem + m[7]);
    const int p = m[3];
    T* y = reinterpret_cast<T*>(pick3(a.y, p));
    const int64_t ystr = pick3(a.y_stride, p);
    const T* dg = INBAND ? reinterpret_cast<const T*>(pick3(a.delta, p)) + delta_off : nullptr;
    const int64_t dgs = a.delta_stride;
    if (m[4] == kPipeChunk) {  // complete chunk: no bounds checks
      switch (m[2]) {
        case 8: expand_stage<T, 1, true, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 16: expand_stage<T, 2, true, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 32: expand_stage<T, 4, true, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 64: expand_stage<T, 8, true, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        default: expand_stage<T, 16, true, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
      }
    } else {
      switch (m[2]) {
        case 8: expand_stage<T, 1, false, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 16: expand_stage<T, 2, false, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 32: expand_stage<T, 4, false, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        case 64: expand_stage<T, 8, false, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
        default: expand_stage<T, 16, false, INBAND>(bs, m, y, ystr, lane, cw, dg, dgs, a.status, &c.tp_gave_up); break;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
}

// INBAND: the instantiation for tensor parallelism with in-band signalling (TpLink::inband); the plain one carries
// none of its checks.
template <typename T, bool EXACT, bool INBAND = false>
__global__ void __launch_bounds__(kPipeThreads, kPipeCtasPerSm) lora_expand_pipe_kernel(const ExpandArgs a) {
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(16) PipeCtl ctl;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (segments_all_elsewhere(a.src, a.tb)) return;
  pipe_init(ctl, tid);
  pdl_launch_dependents();
  if (EXACT) {
    fill_item_counts(a.src, a.tb, ctl, tid, [&](int rr, int) { return expand_items_of(a, rr); });
    __syncthreads();
  }
  if (warp < kProducerWarps) {
    expand_producer<T, EXACT>(a, ring_mem, ctl, lane, warp);
  } else {
    expand_consumer<T, INBAND>(a, ring_mem, ctl, lane, warp - kProducerWarps);
  }
  if (a.tp.enabled && a.tp.inband != 3) {  // (rotating thirds: nothing to do at the end of an expand)
    if (INBAND) {
      // what this exchange used of its half of the delta buffer: [nproj][full_tokens][delta_stride] elements from
      // delta[0] on
      tp_inband_finish(a.tp, const_cast<void*>(a.delta[0]),
                       a.nproj * a.tp.full_tokens * a.delta_stride * static_cast<int64_t>(sizeof(T)));
    } else {
      tp_link_finish(a.tp, false);
    }
  }
}

}  // namespace slora
