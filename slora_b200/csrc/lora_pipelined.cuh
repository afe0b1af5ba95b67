// Persistent, warp-specialised, mbarrier-pipelined LoRA shrink / expand kernels (the fast path).
//
// One CTA per SM walks its share of the work items (item i belongs to CTA i mod gridDim.x).  Warp 0 is the
// producer: its 32 lanes resolve 32 upcoming items in parallel (tile record -> table entries -> row addresses and
// token ids), then feed a ring of kPipeStages shared-memory stages with bulk asynchronous copies
// (cp.async.bulk + mbarrier complete_tx), one lane per copy.  Warps 1..4 are consumers: they wait on a stage's
// "full" barrier, do the arithmetic and release the stage through its "empty" barrier.  Consumer warps never
// synchronise with each other (shrink: one adapter row per warp; expand: one 2048-element span of the B chunk per
// warp), so every wait in the kernel is an mbarrier wait with a time limit.
//
// Programmatic dependent launch: the producer fills the first stages with adapter rows (which no kernel on the
// stream writes) before it executes griddepcontrol.wait, and only then requests activations (x, y, delta).  With a
// ring of ~100 KB two kernels fit on an SM, so the next kernel's prologue overlaps this kernel's tail.
//
// Shrink stage  = K-chunk of 1024 elements: [4 adapter rows][8 token rows] (24 KB); an item is (tile, projection,
//                 block of 4 rows) and spans ceil(h_in / 1024) consecutive stages; accumulators stay in registers.
// Expand stage  = one item (tile half of <= 4 tokens, projection, 8192-element chunk of B): [B chunk 16 KB]
//                 [y segments 4 x 2 KB][delta rows 4 x 256 B] (25 KB).  y is read through the stage and written
//                 back with plain coalesced stores.
#pragma once

#include "lora_common.cuh"

namespace slora {

constexpr int kPipeStages = 4;
constexpr int kConsumerWarps = 4;
constexpr int kPipeThreads = 32 * (1 + kConsumerWarps);
constexpr int kKC = 1024;  // K elements per shrink stage
constexpr int kShrinkStageBytes = (kMaxRows + kTileTokens) * kKC * 2;
constexpr int kHalfTokens = 4;  // tokens per expand item
constexpr int kYSlot = kChunk / 8;  // outputs per token in a stage (r = 8 gives the most)
constexpr int kExpandYBytes = kHalfTokens * kYSlot * 2;
constexpr int kExpandDBytes = kHalfTokens * 128 * 2;
constexpr int kExpandStageBytes = kChunk * 2 + kExpandYBytes + kExpandDBytes;
constexpr int kMaxPieces = 8;  // B copies per expand stage (lanes 0..7); y copies use lanes 8..11, delta 12..15
constexpr int kSpanRows = 4;   // pool rows a B chunk may touch

constexpr int FLAG_FIRST = 1, FLAG_LAST = 2, FLAG_END = 4;
constexpr uint32_t FULL_MASK = 0xffffffffu;
constexpr uint64_t kWaitNs = 1000000000ull;  // one second

__device__ __forceinline__ uint64_t gtime_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Wait for a barrier phase for at most kWaitNs; false on timeout.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = gtime_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (gtime_ns() - t0 > kWaitNs) return false;
  }
}

template <typename P>
__device__ __forceinline__ P pick3(P const (&arr)[3], int p) {
  return p == 0 ? arr[0] : (p == 1 ? arr[1] : arr[2]);
}

// ------------------------------------------------------------------------------------------------------------
// shrink
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void shrink_producer(const ShrinkArgs& a, unsigned char* stage_mem, uint64_t* full,
                                                uint64_t* empty, int (*smeta)[16], int lane) {
  const int per_tile = a.nproj * a.max_rb;
  const int64_t n_items = static_cast<int64_t>(tile_count(a.src)) * per_tile;
  const int h_in = a.h_in;
  const int nk = (h_in + kKC - 1) / kKC;
  const int64_t S = a.tb.pool_stride;
  const T* w = reinterpret_cast<const T*>(a.w);
  const T* x = reinterpret_cast<const T*>(a.x);
  const int64_t G = gridDim.x;
  uint32_t g = 0;
  bool waited = false, dead = false;

  for (int64_t batch0 = blockIdx.x; batch0 < n_items && !dead; batch0 += 32 * G) {
    // ---- 32 items resolved in parallel, one per lane ----
    const int64_t item = batch0 + lane * G;
    int m_valid = 0, m_n = 0, m_nrows = 0, m_j0 = 0, m_p = 0;
    int m_tok[kTileTokens];
    int64_t m_row[kMaxRows];
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) m_tok[i] = 0;
#pragma unroll
    for (int j = 0; j < kMaxRows; ++j) m_row[j] = 0;
    if (item < n_items) {
      const int tile = static_cast<int>(item / per_tile);
      const int rem = static_cast<int>(item - static_cast<int64_t>(tile) * per_tile);
      const int p = rem / a.max_rb, rb = rem - p * a.max_rb;
      TileInfo t;
      if (lookup_tile(a.src, a.tb, tile, t, a.status)) {
        const int j0 = rb * kMaxRows;
        if (j0 < t.r) {
          const int nrows = min(kMaxRows, t.r - j0);
          const int64_t base = t.loc_base + static_cast<int64_t>(t.r) * pick3(a.qkvo, p);
          bool ok = true;
#pragma unroll
          for (int j = 0; j < kMaxRows; ++j) {
            if (j < nrows) {
              const int64_t f = static_cast<int64_t>(j0 + j) * h_in;
              const int64_t pr = f / S, col = f - pr * S;
              const int64_t e = pr < t.r ? a.tb.loc[base + pr] : -1;
              if (e < 0 || e >= a.tb.pool_rows) ok = false;
              m_row[j] = e * S + col;
            }
          }
          if (ok) {
#pragma unroll
            for (int i = 0; i < kTileTokens; ++i) {
              if (i < t.n) m_tok[i] = tile_token(t, i);
            }
            m_valid = 1;
            m_n = t.n;
            m_nrows = nrows;
            m_j0 = j0;
            m_p = p;
          } else {
            set_status(a.status, SLORA_STATUS_BAD_TABLE);
          }
        }
      }
    }

    // ---- feed the ring: stages [lo, hi) of this batch, adapter rows (do_w) and/or activations (do_x) ----
    auto emit = [&](uint32_t g0, uint32_t lo, uint32_t hi, bool do_w, bool do_x) -> uint32_t {
      uint32_t gg = g0;
      for (int k = 0; k < 32; ++k) {
        if (!__shfl_sync(FULL_MASK, m_valid, k)) continue;
        const int n = __shfl_sync(FULL_MASK, m_n, k);
        const int nrows = __shfl_sync(FULL_MASK, m_nrows, k);
        const int j0 = __shfl_sync(FULL_MASK, m_j0, k);
        const int p = __shfl_sync(FULL_MASK, m_p, k);
        int64_t myrow = 0;
        int mytok = 0;
#pragma unroll
        for (int j = 0; j < kMaxRows; ++j) {
          const int64_t v = __shfl_sync(FULL_MASK, m_row[j], k);
          if (lane == j) myrow = v;
        }
#pragma unroll
        for (int i = 0; i < kTileTokens; ++i) {
          const int v = __shfl_sync(FULL_MASK, m_tok[i], k);
          if (lane == kMaxRows + i) mytok = v;
        }
        for (int kc = 0; kc < nk; ++kc, ++gg) {
          if (gg < lo || gg >= hi || dead) continue;
          const int s = gg % kPipeStages;
          const uint32_t round = gg / kPipeStages;
          const int klen = min(kKC, h_in - kc * kKC);
          const uint32_t bytes = static_cast<uint32_t>(klen) * sizeof(T);
          T* st = reinterpret_cast<T*>(stage_mem + static_cast<size_t>(s) * kShrinkStageBytes);
          if (do_w) {
            if (round > 0 && !mbar_wait_timed(&empty[s], (round - 1) & 1)) {
              dead = true;
              continue;
            }
            if (lane == 0) {
              smeta[s][0] = (kc == 0 ? FLAG_FIRST : 0) | (kc == nk - 1 ? FLAG_LAST : 0);
              smeta[s][1] = nrows;
              smeta[s][2] = n;
              smeta[s][3] = j0;
              smeta[s][4] = p;
              smeta[s][5] = klen;
            }
            if (lane >= kMaxRows && lane < kMaxRows + kTileTokens) smeta[s][8 + lane - kMaxRows] = mytok;
            __syncwarp();
            if (lane == 0) mbar_expect_tx(&full[s], static_cast<uint32_t>(nrows + n) * bytes);
            __syncwarp();
            if (lane < nrows) bulk_g2s(st + lane * kKC, w + myrow + static_cast<int64_t>(kc) * kKC, bytes, &full[s]);
          }
          if (do_x && lane >= kMaxRows && lane < kMaxRows + n) {
            bulk_g2s(st + lane * kKC, x + static_cast<int64_t>(mytok) * a.x_stride + static_cast<int64_t>(kc) * kKC,
                     bytes, &full[s]);
          }
        }
      }
      return gg;
    };

    if (!waited) {
      // prologue: adapter rows of the first ring-full of stages go out before the grid dependency resolves
      emit(0, 0, kPipeStages, true, false);
      pdl_wait();
      waited = true;
      emit(0, 0, kPipeStages, false, true);
      g = emit(0, kPipeStages, 0xffffffffu, true, true);
    } else {
      g = emit(g, 0, 0xffffffffu, true, true);
    }
  }
  if (dead) {
    if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
    return;
  }
  // end marker
  const int s = g % kPipeStages;
  const uint32_t round = g / kPipeStages;
  if (round > 0 && !mbar_wait_timed(&empty[s], (round - 1) & 1)) {
    if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
    return;
  }
  if (lane == 0) {
    smeta[s][0] = FLAG_END;
    mbar_arrive(&full[s]);
  }
}

template <typename T>
__device__ __forceinline__ void shrink_consumer(const ShrinkArgs& a, const unsigned char* stage_mem, uint64_t* full,
                                                uint64_t* empty, int (*smeta)[16], int lane, int cw) {
  pdl_wait();
  float acc[kTileTokens];
#pragma unroll
  for (int i = 0; i < kTileTokens; ++i) acc[i] = 0.f;
  for (uint32_t g = 0;; ++g) {
    const int s = g % kPipeStages;
    if (!mbar_wait_timed(&full[s], (g / kPipeStages) & 1)) {
      if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
      return;
    }
    const int* m = smeta[s];
    const int flags = m[0];
    if (flags & FLAG_END) return;
    const int nrows = m[1], n = m[2], klen = m[5];
    if (cw < nrows) {
      const T* st = reinterpret_cast<const T*>(stage_mem + static_cast<size_t>(s) * kShrinkStageBytes);
      const T* wrow = st + cw * kKC;
      const T* xs = st + kMaxRows * kKC;
      if (flags & FLAG_FIRST) {
#pragma unroll
        for (int i = 0; i < kTileTokens; ++i) acc[i] = 0.f;
      }
      for (int k = lane * 8; k < klen; k += 256) {
        float wf[8];
        cvt8<T>(*reinterpret_cast<const uint4*>(wrow + k), wf);
#pragma unroll
        for (int i = 0; i < kTileTokens; ++i) {
          if (i < n) {
            float xf[8];
            cvt8<T>(*reinterpret_cast<const uint4*>(xs + i * kKC + k), xf);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[i] = fmaf(wf[e], xf[e], acc[i]);
          }
        }
      }
      if (flags & FLAG_LAST) {
        const int j = m[3] + cw;
        const float tot = warp_reduce_scatter<kTileTokens>(acc, lane);  // lane l: token l >> 2
        const int i = lane >> 2;
        if ((lane & 3) == 0 && i < n && j < a.delta_width) {
          T* d = reinterpret_cast<T*>(pick3(a.delta, m[4]));
          d[static_cast<int64_t>(m[8 + i]) * a.delta_stride + j] = from_f32<T>(tot);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPipeThreads) lora_shrink_pipe_kernel(const ShrinkArgs a) {
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ __align__(8) uint64_t full[kPipeStages];
  __shared__ __align__(8) uint64_t empty[kPipeStages];
  __shared__ int smeta[kPipeStages][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kPipeStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_launch_dependents();
  if (warp == 0) {
    shrink_producer<T>(a, stage_mem, full, empty, smeta, lane);
  } else {
    shrink_consumer<T>(a, stage_mem, full, empty, smeta, lane, warp - 1);
  }
}

// ------------------------------------------------------------------------------------------------------------
// expand
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void expand_producer(const ExpandArgs& a, unsigned char* stage_mem, uint64_t* full,
                                                uint64_t* empty, int (*smeta)[16], int lane) {
  const int total_chunks = a.chunk_begin[a.nproj];
  const int per_tile = 2 * total_chunks;
  const int64_t n_items = static_cast<int64_t>(tile_count(a.src)) * per_tile;
  const int64_t S = a.tb.pool_stride;
  const T* w = reinterpret_cast<const T*>(a.w);
  const int64_t G = gridDim.x;
  uint32_t g = 0;
  bool waited = false, dead = false;

  for (int64_t batch0 = blockIdx.x; batch0 < n_items && !dead; batch0 += 32 * G) {
    const int64_t item = batch0 + lane * G;
    int m_valid = 0, m_nt = 0, m_r = 0, m_p = 0, m_clen = 0, m_obase = 0, m_c0 = 0, m_pr0 = 0;
    float m_scale = 0.f;
    int m_tok[kHalfTokens];
    int64_t m_e[kSpanRows];
#pragma unroll
    for (int i = 0; i < kHalfTokens; ++i) m_tok[i] = 0;
#pragma unroll
    for (int j = 0; j < kSpanRows; ++j) m_e[j] = 0;
    if (item < n_items) {
      const int tile = static_cast<int>(item / per_tile);
      const int rem = static_cast<int>(item - static_cast<int64_t>(tile) * per_tile);
      const int half = rem / total_chunks;
      int c = rem - half * total_chunks;
      int p = 0;
      while (p + 1 < a.nproj && c >= a.chunk_begin[p + 1]) ++p;
      c -= a.chunk_begin[p];
      TileInfo t;
      if (lookup_tile(a.src, a.tb, tile, t, a.status) && half * kHalfTokens < t.n) {
        const int r = t.r * a.rank_mult;
        const int h_out = pick3(a.h_out, p);
        const int64_t flat_total = static_cast<int64_t>(h_out) * r;
        const int64_t c0 = static_cast<int64_t>(c) * kChunk;
        if (c0 < flat_total) {
          if (r != 8 && r != 16 && r != 32 && r != 64 && r != 128) {
            set_status(a.status, SLORA_STATUS_BAD_RANK);
          } else {
            const int clen = static_cast<int>(min(static_cast<int64_t>(kChunk), flat_total - c0));
            const int64_t base = t.loc_base + static_cast<int64_t>(t.r) * pick3(a.qkvo, p);
            const int64_t pr0 = c0 / S, pr1 = (c0 + clen - 1) / S;
            bool ok = pr1 - pr0 < kSpanRows && pr1 < t.r;
            if (ok) {
#pragma unroll
              for (int j = 0; j < kSpanRows; ++j) {
                if (pr0 + j <= pr1) {
                  const int64_t e = a.tb.loc[base + pr0 + j];
                  if (e < 0 || e >= a.tb.pool_rows) ok = false;
                  m_e[j] = e;
                }
              }
            }
            if (ok) {
              m_nt = min(kHalfTokens, t.n - half * kHalfTokens);
#pragma unroll
              for (int i = 0; i < kHalfTokens; ++i) {
                if (i < m_nt) m_tok[i] = tile_token(t, half * kHalfTokens + i);
              }
              m_valid = 1;
              m_r = r;
              m_p = p;
              m_clen = clen;
              m_c0 = static_cast<int>(c0);
              m_obase = static_cast<int>(c0 / r);
              m_pr0 = static_cast<int>(pr0);
              m_scale = to_f32<T>(reinterpret_cast<const T*>(a.scales)[t.adapter]);
            } else {
              set_status(a.status, SLORA_STATUS_BAD_TABLE);
            }
          }
        }
      }
    }

    auto emit = [&](uint32_t g0, uint32_t lo, uint32_t hi, bool do_w, bool do_x) -> uint32_t {
      uint32_t gg = g0;
      for (int k = 0; k < 32; ++k) {
        if (!__shfl_sync(FULL_MASK, m_valid, k)) continue;
        const uint32_t cur = gg++;
        if (cur < lo || cur >= hi || dead) continue;
        const int nt = __shfl_sync(FULL_MASK, m_nt, k);
        const int r = __shfl_sync(FULL_MASK, m_r, k);
        const int p = __shfl_sync(FULL_MASK, m_p, k);
        const int clen = __shfl_sync(FULL_MASK, m_clen, k);
        const int obase = __shfl_sync(FULL_MASK, m_obase, k);
        const int c0 = __shfl_sync(FULL_MASK, m_c0, k);
        const int pr0 = __shfl_sync(FULL_MASK, m_pr0, k);
        const float scale = __shfl_sync(FULL_MASK, m_scale, k);
        int64_t e[kSpanRows];
#pragma unroll
        for (int j = 0; j < kSpanRows; ++j) e[j] = __shfl_sync(FULL_MASK, m_e[j], k);
        int mytok = 0;
#pragma unroll
        for (int i = 0; i < kHalfTokens; ++i) {
          const int v = __shfl_sync(FULL_MASK, m_tok[i], k);
          if ((lane & 3) == i) mytok = v;  // lanes 8..11 (y) and 12..15 (delta) pick token lane & 3
        }
        const int s = cur % kPipeStages;
        const uint32_t round = cur / kPipeStages;
        const int nout = clen / r;
        unsigned char* st = stage_mem + static_cast<size_t>(s) * kExpandStageBytes;
        if (do_w) {
          if (round > 0 && !mbar_wait_timed(&empty[s], (round - 1) & 1)) {
            dead = true;
            continue;
          }
          if (lane == 0) {
            smeta[s][0] = 0;
            smeta[s][1] = nt;
            smeta[s][2] = r;
            smeta[s][3] = p;
            smeta[s][4] = clen;
            smeta[s][5] = obase;
            smeta[s][6] = __float_as_int(scale);
          }
          if (lane >= 8 && lane < 8 + kHalfTokens) smeta[s][lane] = mytok;
          __syncwarp();
          if (lane == 0) {
            mbar_expect_tx(&full[s], static_cast<uint32_t>(clen) * sizeof(T) +
                                         static_cast<uint32_t>(nt) * static_cast<uint32_t>(nout + r) * sizeof(T));
          }
          __syncwarp();
          const int off = lane * a.piece;
          if (lane < kMaxPieces && off < clen) {
            const int64_t f = static_cast<int64_t>(c0) + off;
            const int64_t pr = f / S, col = f - pr * S;
            const int d = static_cast<int>(pr) - pr0;
            const int64_t row = d == 0 ? e[0] : (d == 1 ? e[1] : (d == 2 ? e[2] : e[3]));
            bulk_g2s(st + static_cast<size_t>(off) * sizeof(T), w + row * S + col,
                     static_cast<uint32_t>(min(a.piece, clen - off)) * sizeof(T), &full[s]);
          }
        }
        if (do_x) {
          if (lane >= 8 && lane < 8 + nt) {
            const T* y = reinterpret_cast<const T*>(pick3(a.y, p));
            bulk_g2s(st + kChunk * 2 + (lane - 8) * kYSlot * 2,
                     y + static_cast<int64_t>(mytok) * pick3(a.y_stride, p) + obase,
                     static_cast<uint32_t>(nout) * sizeof(T), &full[s]);
          } else if (lane >= 12 && lane < 12 + nt) {
            const T* d = reinterpret_cast<const T*>(pick3(a.delta, p));
            bulk_g2s(st + kChunk * 2 + kExpandYBytes + (lane - 12) * 256,
                     d + static_cast<int64_t>(mytok) * a.delta_stride, static_cast<uint32_t>(r) * sizeof(T),
                     &full[s]);
          }
        }
      }
      return gg;
    };

    if (!waited) {
      emit(0, 0, kPipeStages, true, false);
      pdl_wait();
      waited = true;
      emit(0, 0, kPipeStages, false, true);
      g = emit(0, kPipeStages, 0xffffffffu, true, true);
    } else {
      g = emit(g, 0, 0xffffffffu, true, true);
    }
  }
  if (dead) {
    if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
    return;
  }
  const int s = g % kPipeStages;
  const uint32_t round = g / kPipeStages;
  if (round > 0 && !mbar_wait_timed(&empty[s], (round - 1) & 1)) {
    if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
    return;
  }
  if (lane == 0) {
    smeta[s][0] = FLAG_END;
    mbar_arrive(&full[s]);
  }
}

// One consumer warp's part of an expand stage.  LPO = lanes per output = r / 8.  The warp owns flat elements
// [cw*2048, +2048) of the chunk as 8 loads of 256 elements; load m, lane l holds the 8 values of output
// (cw*8 + m)*(32/LPO) + l/LPO for k in [(l % LPO)*8, +8).
template <typename T, int LPO>
__device__ __forceinline__ void expand_stage(const T* bs, const T* ys, const T* ds, const int* m, T* y,
                                             int64_t y_stride, int h_out, int lane, int cw) {
  constexpr int OPL = 32 / LPO;
  constexpr int NV = LPO >= 8 ? 1 : 8 / LPO;
  const int nt = m[1], clen = m[4], obase = m[5];
  const float scale = __int_as_float(m[6]);
  float bf[8][8];
#pragma unroll
  for (int mm = 0; mm < 8; ++mm) {
    const int foff = cw * (kChunk / kConsumerWarps) + mm * 256 + lane * 8;
    if (foff < clen) {
      cvt8<T>(*reinterpret_cast<const uint4*>(bs + foff), bf[mm]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) bf[mm][e] = 0.f;
    }
  }
  const int kp = (lane & (LPO - 1)) * 8;
  const int g = lane / LPO;
  const int m_base = expand_m_base<LPO>(lane);
  const bool writer = (LPO < 16) || ((lane & 8) == 0);
  int o_loc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o_loc[i] = (cw * 8 + m_base + i) * OPL + g;  // output index inside the chunk

  for (int tt = 0; tt < nt; ++tt) {
    float d[8];
    cvt8<T>(*reinterpret_cast<const uint4*>(ds + tt * 128 + kp), d);
    float v[8];
#pragma unroll
    for (int mm = 0; mm < 8; ++mm) {
      float sacc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) sacc = fmaf(bf[mm][e], d[e], sacc);
      v[mm] = sacc;
    }
    expand_butterfly<LPO>(v, lane);
    T* yrow = y + static_cast<int64_t>(m[8 + tt]) * y_stride + obase;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (writer && obase + o_loc[i] < h_out) {
        yrow[o_loc[i]] = from_f32<T>(to_f32<T>(ys[tt * kYSlot + o_loc[i]]) + scale * v[i]);
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void expand_consumer(const ExpandArgs& a, const unsigned char* stage_mem, uint64_t* full,
                                                uint64_t* empty, int (*smeta)[16], int lane, int cw) {
  pdl_wait();
  for (uint32_t g = 0;; ++g) {
    const int s = g % kPipeStages;
    if (!mbar_wait_timed(&full[s], (g / kPipeStages) & 1)) {
      if (lane == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
      return;
    }
    const int* m = smeta[s];
    if (m[0] & FLAG_END) return;
    const unsigned char* st = stage_mem + static_cast<size_t>(s) * kExpandStageBytes;
    const T* bs = reinterpret_cast<const T*>(st);
    const T* ys = reinterpret_cast<const T*>(st + kChunk * 2);
    const T* ds = reinterpret_cast<const T*>(st + kChunk * 2 + kExpandYBytes);
    const int p = m[3];
    T* y = reinterpret_cast<T*>(pick3(a.y, p));
    const int64_t ystr = pick3(a.y_stride, p);
    const int h_out = pick3(a.h_out, p);
    switch (m[2]) {
      case 8: expand_stage<T, 1>(bs, ys, ds, m, y, ystr, h_out, lane, cw); break;
      case 16: expand_stage<T, 2>(bs, ys, ds, m, y, ystr, h_out, lane, cw); break;
      case 32: expand_stage<T, 4>(bs, ys, ds, m, y, ystr, h_out, lane, cw); break;
      case 64: expand_stage<T, 8>(bs, ys, ds, m, y, ystr, h_out, lane, cw); break;
      default: expand_stage<T, 16>(bs, ys, ds, m, y, ystr, h_out, lane, cw); break;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPipeThreads) lora_expand_pipe_kernel(const ExpandArgs a) {
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ __align__(8) uint64_t full[kPipeStages];
  __shared__ __align__(8) uint64_t empty[kPipeStages];
  __shared__ int smeta[kPipeStages][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kPipeStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  pdl_launch_dependents();
  if (warp == 0) {
    expand_producer<T>(a, stage_mem, full, empty, smeta, lane);
  } else {
    expand_consumer<T>(a, stage_mem, full, empty, smeta, lane, warp - 1);
  }
}

}  // namespace slora
