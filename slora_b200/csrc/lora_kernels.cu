// Multi-adapter LoRA shrink / expand for B200 (sm_100a): device kernels and the C ABI around them.
//
// What is computed (the reference's math, slora/csrc/bgmv/bgmv_impl.cuh:15-149 and :153-208):
//   shrink: delta[t, j] = sum_k x[t, k] * A_a[j, k]                   j < r_a,  a = adapter of token t
//   expand: y[t, o]    += scale_a * sum_k delta[t, k] * B_a[o, k]     k < r_a
// with A_a / B_a read in place from the paged pool through the start / ranks4 / loc tables.
//
// How it is organised here (not the reference's one-CTA-per-(token,row) scheme):
//   * a work item is (tile, projection, sub-block).  A tile is up to 8 tokens that use the same adapter
//     (built once per batch by plan_build_kernel), so adapter rows are fetched once per tile, not once per token;
//   * adapter rows are contiguous 16-byte-aligned runs in the pool, so each CTA stages them into shared memory
//     with bulk asynchronous copies (cp.async.bulk + mbarrier) issued before the kernel waits for its
//     predecessor on the stream (programmatic dependent launch): the weight stream of one kernel overlaps the
//     tail of the previous one;
//   * the shrink reduces over h_in with a register tile [rows x tokens] per thread, a warp-shuffle
//     reduce-scatter and one shared-memory hop across the four warps;
//   * the expand keeps a 16 KB chunk of B in registers as fp32, reads each token's (pre-scaled) delta from shared
//     memory and reduces across the r/8 lanes that share an output with a shuffle butterfly, so every lane ends
//     up owning distinct outputs for the read-modify-write of y.
// Every wait on an mbarrier is bounded; on timeout the CTA records SLORA_STATUS_TIMEOUT and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "slora_b200.h"

namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kTileTokens = 8;   // tokens per tile (plan granularity)
constexpr int kMaxRows = 4;      // A rows staged per shrink CTA (upper bound)
constexpr int kTokPass = 4;      // tokens reduced per register pass in the shrink
constexpr int kChunk = 8192;     // flat B elements per expand CTA (16 KB)
constexpr int kWarpSpan = kChunk / kWarps;  // 2048 elements per warp
constexpr int kShrinkSmemBudget = 64 * 1024;
constexpr uint32_t kSpinLimit = 1u << 18;

// plan workspace: int32 words
constexpr int PH_MAGIC = 0, PH_NTILES = 1, PH_STATUS = 2, PH_MAXTILES = 3, PH_T = 4, PH_NADAPTERS = 5;
constexpr int PH_WORDS = 16;
constexpr int32_t kPlanMagic = 0x534c5031;  // "SLP1"

enum TileMode { MODE_TOKEN = 0, MODE_PLAN = 1, MODE_SEGMENT = 2 };

struct TileSrc {
  const int32_t* plan;
  const int64_t* ids;        // TOKEN: per token; SEGMENT: per segment
  const int32_t* seg_start;
  const int32_t* seg_len;
  int mode;
  int n_seg;
  int tiles_per_seg;
  int64_t T;
};

struct Tile {
  int64_t adapter;
  int n;
  int first;
  const int32_t* perm;
};

struct Tables {
  const int64_t* start;
  const int64_t* ranks4;
  const int64_t* loc;
  int64_t n_adapters;
  int64_t loc_len;
  int64_t pool_rows;
  int64_t pool_stride;
};

struct ShrinkArgs {
  TileSrc src;
  Tables tb;
  const void* w;
  const void* x;
  int64_t x_stride;
  int h_in;
  void* delta[3];
  int qkvo[3];
  int nproj;
  int64_t delta_stride;
  int delta_width;
  int max_rb;        // row blocks enumerated per (tile, projection)
  int rows_per_cta;  // <= kMaxRows
  int tok_pass;      // <= kTokPass, tokens staged per pass
  int piece;         // elements per bulk copy (divides h_in; a piece never straddles a pool row)
  int32_t* status;
};

struct ExpandArgs {
  TileSrc src;
  Tables tb;
  const void* w;
  const void* scales;
  void* y[3];
  int64_t y_stride[3];
  int h_out[3];
  const void* delta[3];
  int qkvo[3];
  int chunk_begin[4];  // prefix sums of chunks per projection
  int nproj;
  int64_t delta_stride;
  int delta_parts;
  int64_t delta_part_stride;
  int rank_mult;
  int piece;  // elements per bulk copy (power of two dividing pool_stride, <= kChunk)
  int32_t* status;
};

// ------------------------------------------------------------------------------------------------------------
// PTX helpers
// ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: true when the phase completed within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// Bulk asynchronous copy global -> this CTA's shared memory; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <typename T>
__device__ __forceinline__ void cvt8(const uint4& v, float (&f)[8]);
template <>
__device__ __forceinline__ void cvt8<__half>(const uint4& v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void cvt8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void set_status(int32_t* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

// Which tokens / adapter does tile `tile_idx` cover?  Uniform across the CTA.
__device__ __forceinline__ bool resolve_tile(const TileSrc& s, int tile_idx, Tile& t) {
  if (s.mode == MODE_PLAN) {
    const int32_t* hdr = s.plan;
    if (tile_idx >= hdr[PH_NTILES]) return false;
    const int4 rec = reinterpret_cast<const int4*>(s.plan + PH_WORDS)[tile_idx];
    t.adapter = rec.x;
    t.first = rec.y;
    t.n = rec.z;
    t.perm = s.plan + PH_WORDS + 4 * hdr[PH_MAXTILES];
    return t.n > 0;
  }
  if (s.mode == MODE_TOKEN) {
    if (tile_idx >= s.T) return false;
    t.adapter = s.ids[tile_idx];
    t.first = tile_idx;
    t.n = 1;
    t.perm = nullptr;
    return true;
  }
  const int seg = tile_idx / s.tiles_per_seg;
  const int sub = tile_idx - seg * s.tiles_per_seg;
  if (seg >= s.n_seg) return false;
  const int64_t len = s.seg_len[seg];
  const int64_t off = static_cast<int64_t>(sub) * kTileTokens;
  if (off >= len) return false;
  const int64_t first = static_cast<int64_t>(s.seg_start[seg]) + off;
  if (first < 0 || first >= s.T) return false;
  int64_t n = len - off;
  if (n > kTileTokens) n = kTileTokens;
  if (first + n > s.T) n = s.T - first;
  t.adapter = s.ids[seg];
  t.first = static_cast<int>(first);
  t.n = static_cast<int>(n);
  t.perm = nullptr;
  return true;
}

// Sum V per-lane values across the warp; lane l returns the total of logical index (l >> (5 - log2 V)).
template <int V>
__device__ __forceinline__ float warp_reduce_scatter(float (&v)[V], int lane) {
  int mask = 16;
#pragma unroll
  for (int half = V / 2; half >= 1; half >>= 1) {
    const bool up = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float keep = up ? v[i + half] : v[i];
      const float send = up ? v[i] : v[i + half];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
    mask >>= 1;
  }
#pragma unroll
  for (; mask >= 1; mask >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], mask);
  return v[0];
}

// ------------------------------------------------------------------------------------------------------------
// plan: group the batch's tokens by adapter (one CTA; T and n_adapters are a few thousand at most)
// workspace words: [header PH_WORDS][tiles 4*max_tiles][perm T][pos T][cnt n_adapters]
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) plan_build_kernel(int32_t* ws, const int64_t* __restrict__ ids, int T,
                                                          int n_adapters, int max_tiles) {
  int32_t* hdr = ws;
  int32_t* tiles = ws + PH_WORDS;
  int32_t* perm = tiles + 4 * max_tiles;
  int32_t* pos = perm + T;
  int32_t* cnt = pos + T;
  __shared__ int s_tok[32], s_tile[32];
  __shared__ int s_status;
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < n_adapters; i += nthr) cnt[i] = 0;
  if (tid == 0) s_status = 0;
  __syncthreads();
  for (int t = tid; t < T; t += nthr) {
    const int64_t a = ids[t];
    if (a < 0 || a >= n_adapters) {
      pos[t] = -1;
      s_status = SLORA_STATUS_BAD_ID;
    } else {
      pos[t] = atomicAdd(&cnt[a], 1);
    }
  }
  __syncthreads();
  // exclusive scan over adapters of (tokens, tiles); each thread owns a contiguous run of adapters
  const int per = (n_adapters + nthr - 1) / nthr;
  const int lo = min(tid * per, n_adapters), hi = min(lo + per, n_adapters);
  int tok_sum = 0, tile_sum = 0;
  for (int a = lo; a < hi; ++a) {
    const int c = cnt[a];
    tok_sum += c;
    tile_sum += (c + kTileTokens - 1) / kTileTokens;
  }
  int tok_inc = tok_sum, tile_inc = tile_sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, tok_inc, off);
    const int b = __shfl_up_sync(0xffffffffu, tile_inc, off);
    if (lane >= off) {
      tok_inc += a;
      tile_inc += b;
    }
  }
  if (lane == 31) {
    s_tok[warp] = tok_inc;
    s_tile[warp] = tile_inc;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = nthr >> 5;
    int a = lane < nw ? s_tok[lane] : 0, b = lane < nw ? s_tile[lane] : 0;
    int ai = a, bi = b;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a2 = __shfl_up_sync(0xffffffffu, ai, off);
      const int b2 = __shfl_up_sync(0xffffffffu, bi, off);
      if (lane >= off) {
        ai += a2;
        bi += b2;
      }
    }
    s_tok[lane] = ai - a;  // exclusive
    s_tile[lane] = bi - b;
    if (lane == 31) {
      hdr[PH_NTILES] = bi;
    }
  }
  __syncthreads();
  int tok_off = s_tok[warp] + tok_inc - tok_sum;
  int tile_off = s_tile[warp] + tile_inc - tile_sum;
  for (int a = lo; a < hi; ++a) {
    const int c = cnt[a];
    cnt[a] = tok_off;  // becomes the group's first slot in perm
    for (int i = 0; i * kTileTokens < c; ++i) {
      int4 rec;
      rec.x = a;
      rec.y = tok_off + i * kTileTokens;
      rec.z = min(kTileTokens, c - i * kTileTokens);
      rec.w = 0;
      if (tile_off < max_tiles) reinterpret_cast<int4*>(tiles)[tile_off] = rec;
      ++tile_off;
    }
    tok_off += c;
  }
  __syncthreads();
  for (int t = tid; t < T; t += nthr) {
    const int p = pos[t];
    if (p >= 0) perm[cnt[ids[t]] + p] = t;
  }
  if (tid == 0) {
    hdr[PH_MAGIC] = kPlanMagic;
    hdr[PH_STATUS] = s_status;
    hdr[PH_MAXTILES] = max_tiles;
    hdr[PH_T] = T;
    hdr[PH_NADAPTERS] = n_adapters;
  }
}

// ------------------------------------------------------------------------------------------------------------
// shrink
// dynamic shared memory: [rows_per_cta][h_in] adapter rows, then [tok_pass][h_in] activation rows
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) lora_shrink_kernel(const ShrinkArgs a) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ __align__(8) uint64_t bar_w;
  __shared__ __align__(8) uint64_t bar_x;
  __shared__ float s_red[kWarps][kMaxRows * kTokPass];
  __shared__ int s_tok[kTileTokens];

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int idx = blockIdx.x;
  const int rb = idx % a.max_rb;
  idx /= a.max_rb;
  const int p = idx % a.nproj;
  const int tile_idx = idx / a.nproj;

  Tile t;
  if (!resolve_tile(a.src, tile_idx, t)) return;
  int32_t* status = a.status;
  if (t.adapter < 0 || t.adapter >= a.tb.n_adapters) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_ID);
    return;
  }
  const int64_t r4 = a.tb.ranks4[t.adapter];
  const int64_t st = a.tb.start[t.adapter];
  if (r4 < 0 || st < 0 || st + r4 > a.tb.loc_len || r4 > (int64_t(1) << 20)) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
    return;
  }
  const int r = static_cast<int>(r4 >> 2);
  const int j0 = rb * a.rows_per_cta;
  if (j0 >= r) return;
  const int nrows = min(a.rows_per_cta, r - j0);
  const int64_t base = st + static_cast<int64_t>(r) * a.qkvo[p];
  const int h_in = a.h_in;
  const int64_t S = a.tb.pool_stride;
  T* ws = reinterpret_cast<T*>(dyn_smem);
  T* xs = ws + static_cast<size_t>(a.rows_per_cta) * h_in;

  if (tid == 0) {
    mbar_init(&bar_w, 1);
    mbar_init(&bar_x, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  // every bulk copy ("piece") is checked before any is issued
  const int ppr = h_in / a.piece;  // pieces per A row
  const int npieces = nrows * ppr;
  bool ok = true;
  for (int i = tid; i < npieces; i += kThreads) {
    const int j = i / ppr, q = i - j * ppr;
    const int64_t f = static_cast<int64_t>(j0 + j) * h_in + static_cast<int64_t>(q) * a.piece;
    const int64_t pr = f / S;
    if (pr >= r) {
      ok = false;
    } else {
      const int64_t e = a.tb.loc[base + pr];
      if (e < 0 || e >= a.tb.pool_rows) ok = false;
    }
  }
  if (!__syncthreads_and(ok)) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
    return;
  }
  if (tid == 0) mbar_expect_tx(&bar_w, static_cast<uint32_t>(nrows) * h_in * sizeof(T));
  __syncthreads();
  for (int i = tid; i < npieces; i += kThreads) {
    const int j = i / ppr, q = i - j * ppr;
    const int64_t f = static_cast<int64_t>(j0 + j) * h_in + static_cast<int64_t>(q) * a.piece;
    const int64_t pr = f / S, col = f - pr * S;
    const int64_t e = a.tb.loc[base + pr];
    bulk_g2s(ws + static_cast<size_t>(j) * h_in + static_cast<size_t>(q) * a.piece,
             reinterpret_cast<const T*>(a.w) + e * S + col, a.piece * sizeof(T), &bar_w);
  }
  if (tid < t.n) s_tok[tid] = t.perm ? t.perm[t.first + tid] : t.first + tid;

  // everything above touches only the pool and the tables; activations and delta come after the wait
  pdl_wait();
  __syncthreads();

  uint32_t xphase = 0;
  bool w_ready = false;
  T* dout = reinterpret_cast<T*>(a.delta[p]);
  for (int t0 = 0; t0 < t.n; t0 += a.tok_pass) {
    const int nt = min(a.tok_pass, t.n - t0);
    if (tid == 0) {
      fence_proxy_async();
      mbar_expect_tx(&bar_x, static_cast<uint32_t>(nt) * h_in * sizeof(T));
      for (int i = 0; i < nt; ++i) {
        bulk_g2s(xs + static_cast<size_t>(i) * h_in,
                 reinterpret_cast<const T*>(a.x) + static_cast<int64_t>(s_tok[t0 + i]) * a.x_stride,
                 h_in * sizeof(T), &bar_x);
      }
    }
    bool arrived = true;
    if (!w_ready) {
      arrived = mbar_wait(&bar_w, 0);
      w_ready = true;
    }
    arrived = arrived && mbar_wait(&bar_x, xphase);
    xphase ^= 1;
    if (!__syncthreads_and(arrived)) {
      if (tid == 0) set_status(status, SLORA_STATUS_TIMEOUT);
      // give copies still in flight one more bounded chance to land before this CTA's shared memory is reused
      mbar_wait(&bar_w, 0);
      mbar_wait(&bar_x, xphase ^ 1);
      return;
    }

    float acc[kMaxRows * kTokPass];
#pragma unroll
    for (int i = 0; i < kMaxRows * kTokPass; ++i) acc[i] = 0.f;
    for (int k = tid * 8; k < h_in; k += kThreads * 8) {
      float xf[kTokPass][8];
#pragma unroll
      for (int i = 0; i < kTokPass; ++i) {
        if (i < nt) {
          cvt8<T>(*reinterpret_cast<const uint4*>(xs + static_cast<size_t>(i) * h_in + k), xf[i]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) xf[i][e] = 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxRows; ++j) {
        if (j < nrows) {
          float wf[8];
          cvt8<T>(*reinterpret_cast<const uint4*>(ws + static_cast<size_t>(j) * h_in + k), wf);
#pragma unroll
          for (int i = 0; i < kTokPass; ++i) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[j * kTokPass + i] = fmaf(wf[e], xf[i][e], acc[j * kTokPass + i]);
          }
        }
      }
    }
    const float tot = warp_reduce_scatter<kMaxRows * kTokPass>(acc, lane);
    if ((lane & 1) == 0) s_red[warp][lane >> 1] = tot;
    __syncthreads();
    if (tid < kMaxRows * kTokPass) {
      const int j = tid / kTokPass, i = tid - j * kTokPass;
      if (j < nrows && i < nt && j0 + j < a.delta_width) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += s_red[w][tid];
        dout[static_cast<int64_t>(s_tok[t0 + i]) * a.delta_stride + j0 + j] = from_f32<T>(sum);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------------------
// expand
// ------------------------------------------------------------------------------------------------------------
template <int HALF>
__device__ __forceinline__ void exch(float (&v)[8], int lane, int mask) {
  const bool up = (lane & mask) != 0;
#pragma unroll
  for (int i = 0; i < HALF; ++i) {
    const float keep = up ? v[i + HALF] : v[i];
    const float send = up ? v[i] : v[i + HALF];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
  }
}

// One warp's part of an expand chunk.  LPO = lanes per output = r / 8.
// The warp owns flat elements [warp*2048, +2048) of the chunk as 8 loads of 256 elements; load m, lane l holds the
// 8 values of output (warp*8 + m)*(32/LPO) + l/LPO for k in [(l % LPO)*8, +8).
template <typename T, int LPO>
__device__ __forceinline__ void expand_compute(const T* bs, const float* sd, int n, int r, int clen, int64_t o_base,
                                               T* y, int64_t y_stride, int h_out, const int* s_tok, int lane,
                                               int warp) {
  constexpr int OPL = 32 / LPO;
  constexpr int NV = LPO >= 8 ? 1 : 8 / LPO;  // outputs a lane owns after the butterfly
  float bf[8][8];
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int foff = warp * kWarpSpan + m * 256 + lane * 8;
    if (foff < clen) {
      cvt8<T>(*reinterpret_cast<const uint4*>(bs + foff), bf[m]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) bf[m][e] = 0.f;
    }
  }
  const int kp = (lane & (LPO - 1)) * 8;
  const int g = lane / LPO;
  int m_base = 0;
  if (LPO >= 2) m_base += (lane & 1) ? 4 : 0;
  if (LPO >= 4) m_base += (lane & 2) ? 2 : 0;
  if (LPO >= 8) m_base += (lane & 4) ? 1 : 0;
  const bool writer = (LPO < 16) || ((lane & 8) == 0);
  int64_t o_idx[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o_idx[i] = o_base + static_cast<int64_t>(warp * 8 + m_base + i) * OPL + g;

  for (int tt = 0; tt < n; ++tt) {
    T* yrow = y + static_cast<int64_t>(s_tok[tt]) * y_stride;
    float yv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) yv[i] = (writer && o_idx[i] < h_out) ? to_f32<T>(yrow[o_idx[i]]) : 0.f;
    const float4 d0 = *reinterpret_cast<const float4*>(sd + tt * r + kp);
    const float4 d1 = *reinterpret_cast<const float4*>(sd + tt * r + kp + 4);
    const float d[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    float v[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(bf[m][e], d[e], s);
      v[m] = s;
    }
    if (LPO >= 2) exch<4>(v, lane, 1);
    if (LPO >= 4) exch<2>(v, lane, 2);
    if (LPO >= 8) exch<1>(v, lane, 4);
    if (LPO >= 16) v[0] += __shfl_xor_sync(0xffffffffu, v[0], 8);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (writer && o_idx[i] < h_out) yrow[o_idx[i]] = from_f32<T>(yv[i] + v[i]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) lora_expand_kernel(const ExpandArgs a) {
  __shared__ __align__(128) T bs[kChunk];
  __shared__ __align__(16) float sd[kTileTokens * 128];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_tok[kTileTokens];

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int total_chunks = a.chunk_begin[a.nproj];
  const int tile_idx = blockIdx.x / total_chunks;
  int c = blockIdx.x - tile_idx * total_chunks;
  int p = 0;
  while (p + 1 < a.nproj && c >= a.chunk_begin[p + 1]) ++p;
  c -= a.chunk_begin[p];

  Tile t;
  if (!resolve_tile(a.src, tile_idx, t)) return;
  int32_t* status = a.status;
  if (t.adapter < 0 || t.adapter >= a.tb.n_adapters) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_ID);
    return;
  }
  const int64_t r4 = a.tb.ranks4[t.adapter];
  const int64_t st = a.tb.start[t.adapter];
  if (r4 < 0 || st < 0 || st + r4 > a.tb.loc_len || r4 > (int64_t(1) << 20)) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
    return;
  }
  const int slot = static_cast<int>(r4 >> 2);
  const int r = slot * a.rank_mult;
  if (r == 0) return;
  const int h_out = a.h_out[p];
  const int64_t flat_total = static_cast<int64_t>(h_out) * r;
  const int64_t c0 = static_cast<int64_t>(c) * kChunk;
  if (c0 >= flat_total) return;
  if (r != 8 && r != 16 && r != 32 && r != 64 && r != 128) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_RANK);
    return;
  }
  const int clen = static_cast<int>(min(static_cast<int64_t>(kChunk), flat_total - c0));
  const int64_t base = st + static_cast<int64_t>(slot) * a.qkvo[p];
  const int64_t S = a.tb.pool_stride;

  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  const int npieces = (clen + a.piece - 1) / a.piece;
  bool ok = true;
  for (int i = tid; i < npieces; i += kThreads) {
    const int64_t f = c0 + static_cast<int64_t>(i) * a.piece;
    const int64_t pr = f / S;
    if (pr >= slot) {
      ok = false;
    } else {
      const int64_t e = a.tb.loc[base + pr];
      if (e < 0 || e >= a.tb.pool_rows) ok = false;
    }
  }
  if (!__syncthreads_and(ok)) {
    if (tid == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
    return;
  }
  if (tid == 0) mbar_expect_tx(&bar, static_cast<uint32_t>(clen) * sizeof(T));
  __syncthreads();
  for (int i = tid; i < npieces; i += kThreads) {
    const int64_t f = c0 + static_cast<int64_t>(i) * a.piece;
    const int64_t pr = f / S, col = f - pr * S;
    const int64_t e = a.tb.loc[base + pr];
    const int len = min(a.piece, clen - i * a.piece);
    bulk_g2s(bs + static_cast<size_t>(i) * a.piece, reinterpret_cast<const T*>(a.w) + e * S + col,
             len * sizeof(T), &bar);
  }
  if (tid < t.n) s_tok[tid] = t.perm ? t.perm[t.first + tid] : t.first + tid;
  const float scale = to_f32<T>(reinterpret_cast<const T*>(a.scales)[t.adapter]);

  pdl_wait();
  __syncthreads();

  // this tile's delta rows, pre-multiplied by the adapter's scale
  {
    const T* dsrc = reinterpret_cast<const T*>(a.delta[p]);
    const int rs = r / a.delta_parts;
    const int cnt = t.n * r;
    for (int i = tid; i < cnt; i += kThreads) {
      const int tt = i / r, k = i - tt * r;
      const int part = k / rs, j = k - part * rs;
      sd[i] = scale * to_f32<T>(dsrc[static_cast<int64_t>(part) * a.delta_part_stride +
                                      static_cast<int64_t>(s_tok[tt]) * a.delta_stride + j]);
    }
  }
  const bool arrived = mbar_wait(&bar, 0);
  if (!__syncthreads_and(arrived)) {
    if (tid == 0) set_status(status, SLORA_STATUS_TIMEOUT);
    mbar_wait(&bar, 0);
    return;
  }
  const int64_t o_base = c0 / r;
  T* y = reinterpret_cast<T*>(a.y[p]);
  switch (r) {
    case 8: expand_compute<T, 1>(bs, sd, t.n, r, clen, o_base, y, a.y_stride[p], h_out, s_tok, lane, warp); break;
    case 16: expand_compute<T, 2>(bs, sd, t.n, r, clen, o_base, y, a.y_stride[p], h_out, s_tok, lane, warp); break;
    case 32: expand_compute<T, 4>(bs, sd, t.n, r, clen, o_base, y, a.y_stride[p], h_out, s_tok, lane, warp); break;
    case 64: expand_compute<T, 8>(bs, sd, t.n, r, clen, o_base, y, a.y_stride[p], h_out, s_tok, lane, warp); break;
    default: expand_compute<T, 16>(bs, sd, t.n, r, clen, o_base, y, a.y_stride[p], h_out, s_tok, lane, warp); break;
  }
}

// ------------------------------------------------------------------------------------------------------------
// table check (debug)
// ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void report_bad(int32_t* report, int kind, int64_t index) {
  if (atomicAdd(&report[0], 1) == 0) {
    report[1] = kind;
    report[2] = static_cast<int32_t>(index);
  }
}
__global__ void validate_tables_kernel(const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                                       const int64_t* ids, int64_t n_adapters, int64_t loc_len, int64_t T,
                                       int64_t pool_rows, int32_t* report) {
  const int64_t gid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t gsz = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = gid; i < T; i += gsz) {
    if (ids != nullptr && (ids[i] < 0 || ids[i] >= n_adapters)) report_bad(report, 1, i);
  }
  for (int64_t i = gid; i < n_adapters; i += gsz) {
    const int64_t s = start[i], r4 = ranks4[i];
    if (s < 0 || r4 < 0 || (r4 & 3) != 0 || s + r4 > loc_len) report_bad(report, 2, i);
  }
  for (int64_t i = gid; i < loc_len; i += gsz) {
    if (loc[i] < 0 || loc[i] >= pool_rows) report_bad(report, 3, i);
  }
}
// Empty kernel launched (without programmatic serialization) right after plan_build_kernel: later kernels that
// start early under programmatic dependent launch read the plan before their grid-dependency wait, and this
// fully serialised launch in between guarantees the plan's writes are complete and visible by then.
__global__ void plan_fence_kernel() {}

__global__ void zero_report_kernel(int32_t* report) {
  if (threadIdx.x < 4) report[threadIdx.x] = 0;
}

// ------------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------------
thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int pow2_divisor(int64_t v, int cap) {
  int p = 1;
  while (p * 2 <= cap && v % (p * 2) == 0) p *= 2;
  return p;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return SLORA_OK;
}

int max_tiles_for(int64_t T, int64_t n_adapters) {
  const int64_t groups = T < n_adapters ? T : n_adapters;
  return static_cast<int>((T + kTileTokens - 1) / kTileTokens + groups);
}

struct PlanLayout {
  int max_tiles;
  size_t words;
};
PlanLayout plan_layout(int64_t T, int64_t n_adapters) {
  PlanLayout l;
  l.max_tiles = max_tiles_for(T, n_adapters);
  l.words = static_cast<size_t>(PH_WORDS) + 4u * l.max_tiles + 2u * static_cast<size_t>(T) +
            static_cast<size_t>(n_adapters) + 4;
  return l;
}

int check_common(int dtype, const Tables& tb, const void* w) {
  if (dtype != SLORA_F16 && dtype != SLORA_BF16) return fail(SLORA_ERR_DTYPE, "unsupported dtype %d", dtype);
  if (!w || !tb.start || !tb.ranks4 || !tb.loc) return fail(SLORA_ERR_NULL, "null pool or table pointer");
  if (!aligned16(w)) return fail(SLORA_ERR_ALIGN, "pool buffer is not 16-byte aligned");
  if (tb.pool_stride <= 0 || tb.pool_stride % 8 != 0)
    return fail(SLORA_ERR_SHAPE, "pool_stride=%lld must be a positive multiple of 8", (long long)tb.pool_stride);
  if (tb.pool_rows <= 0 || tb.n_adapters < 0 || tb.loc_len < 0)
    return fail(SLORA_ERR_SHAPE, "negative or zero table/pool size");
  return SLORA_OK;
}

int tile_src_slots(const TileSrc& s, int64_t n_adapters, int* slots) {
  if (s.mode == MODE_PLAN) {
    *slots = max_tiles_for(s.T, n_adapters);
  } else if (s.mode == MODE_TOKEN) {
    *slots = static_cast<int>(s.T);
  } else {
    *slots = s.n_seg * s.tiles_per_seg;
  }
  return SLORA_OK;
}

template <typename K, typename A>
int launch(K kernel, int64_t grid, size_t smem, unsigned flags, cudaStream_t stream, const A& args, const char* what) {
  if (grid <= 0) return SLORA_OK;
  if (grid > 0x7fffffffLL) return fail(SLORA_ERR_SHAPE, "%s: grid of %lld CTAs is too large", what, (long long)grid);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int nattr = 0;
  if (flags & SLORA_FLAG_PDL) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return SLORA_OK;
}

// Opt in to more than 48 KB of dynamic shared memory, once per (kernel, device) and size high-water mark.
template <typename K>
int ensure_dyn_smem(K kernel, int which, size_t smem) {
  static int high_water[2][64];
  if (smem <= 48 * 1024) return SLORA_OK;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (static_cast<int>(smem) <= high_water[which][dev]) return SLORA_OK;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "cudaFuncSetAttribute(%zu bytes): %s", smem, cudaGetErrorString(e));
  }
  high_water[which][dev] = static_cast<int>(smem);
  return SLORA_OK;
}

int run_shrink(const TileSrc& src, const Tables& tb, const void* w, const void* x, int64_t x_stride, int h_in,
               int nproj, const int* qkvo, void* const* delta, int64_t delta_stride, int delta_width, int dtype,
               unsigned flags, int32_t* status, cudaStream_t stream) {
  int rc = check_common(dtype, tb, w);
  if (rc) return rc;
  if (!x) return fail(SLORA_ERR_NULL, "x is null");
  if (nproj < 1 || nproj > 3) return fail(SLORA_ERR_SHAPE, "nproj=%d outside 1..3", nproj);
  if (h_in <= 0 || h_in % 8 != 0 || h_in >= 65536 * 8)
    return fail(SLORA_ERR_SHAPE, "No suitable kernel. h_in=%d must be a positive multiple of 8", h_in);
  if (delta_width <= 0) return fail(SLORA_ERR_SHAPE, "delta_width=%d must be positive", delta_width);
  if (!aligned16(x) || x_stride % 8 != 0) return fail(SLORA_ERR_ALIGN, "x rows are not 16-byte aligned");
  const int64_t S = tb.pool_stride;
  int piece;
  if (S % h_in == 0) {
    piece = h_in;
  } else {
    piece = pow2_divisor(S, h_in);
    if (h_in % piece != 0) piece = pow2_divisor(h_in, piece);
    if (piece < 8) return fail(SLORA_ERR_SHAPE, "pool_stride=%lld and h_in=%d share no 16-byte piece", (long long)S, h_in);
  }
  if (src.T <= 0) return SLORA_OK;
  ShrinkArgs a;
  memset(&a, 0, sizeof(a));
  a.src = src;
  a.tb = tb;
  a.w = w;
  a.x = x;
  a.x_stride = x_stride;
  a.h_in = h_in;
  a.nproj = nproj;
  for (int p = 0; p < nproj; ++p) {
    if (!delta[p]) return fail(SLORA_ERR_NULL, "delta[%d] is null", p);
    if (qkvo[p] < 0 || qkvo[p] > 3) return fail(SLORA_ERR_QKVO, "qkvo=%d outside 0..3", qkvo[p]);
    a.delta[p] = delta[p];
    a.qkvo[p] = qkvo[p];
  }
  a.delta_stride = delta_stride;
  a.delta_width = delta_width;
  const size_t row_bytes = static_cast<size_t>(h_in) * 2;
  int rows = static_cast<int>(kShrinkSmemBudget / 2 / row_bytes);
  rows = rows < 1 ? 1 : (rows > kMaxRows ? kMaxRows : rows);
  if (rows > delta_width) rows = delta_width;
  int toks = static_cast<int>((kShrinkSmemBudget - rows * row_bytes) / row_bytes);
  toks = toks < 1 ? 1 : (toks > kTokPass ? kTokPass : toks);
  if (src.mode == MODE_TOKEN) toks = 1;
  const size_t smem = (static_cast<size_t>(rows) + toks) * row_bytes;
  if (smem > 200 * 1024) return fail(SLORA_ERR_SHAPE, "No suitable kernel. h_in=%d needs %zu bytes of shared memory", h_in, smem);
  a.rows_per_cta = rows;
  a.tok_pass = toks;
  a.piece = piece;
  a.max_rb = (delta_width + rows - 1) / rows;
  a.status = status;
  int slots = 0;
  tile_src_slots(src, tb.n_adapters, &slots);
  const int64_t grid = static_cast<int64_t>(slots) * nproj * a.max_rb;
  if (dtype == SLORA_F16) {
    auto k = lora_shrink_kernel<__half>;
    rc = ensure_dyn_smem(k, 0, smem);
    return rc ? rc : launch(k, grid, smem, flags, stream, a, "shrink");
  }
  auto k = lora_shrink_kernel<__nv_bfloat16>;
  rc = ensure_dyn_smem(k, 1, smem);
  return rc ? rc : launch(k, grid, smem, flags, stream, a, "shrink");
}

int run_expand(const TileSrc& src, const Tables& tb, const void* w, const void* scales, int nproj, const int* qkvo,
               void* const* y, const int64_t* y_stride, const int* h_out, const void* const* delta,
               int64_t delta_stride, int delta_width, int delta_parts, int64_t delta_part_stride, int rank_mult,
               int dtype, unsigned flags, int32_t* status, cudaStream_t stream) {
  int rc = check_common(dtype, tb, w);
  if (rc) return rc;
  if (!scales) return fail(SLORA_ERR_NULL, "scales is null");
  if (nproj < 1 || nproj > 3) return fail(SLORA_ERR_SHAPE, "nproj=%d outside 1..3", nproj);
  if (rank_mult < 1 || delta_parts < 1) return fail(SLORA_ERR_SHAPE, "rank_mult and delta_parts must be >= 1");
  if (delta_width <= 0) return fail(SLORA_ERR_SHAPE, "delta_width=%d must be positive", delta_width);
  const int max_rank = delta_width * delta_parts;  // widest B rank the delta buffer can hold
  if (max_rank > 128) return fail(SLORA_ERR_RANK, "No suitable kernel. rank %d > 128", max_rank);
  const int piece = pow2_divisor(tb.pool_stride, kChunk);
  if (piece < 8) return fail(SLORA_ERR_SHAPE, "pool_stride=%lld is not a multiple of 8", (long long)tb.pool_stride);
  if (src.T <= 0) return SLORA_OK;
  ExpandArgs a;
  memset(&a, 0, sizeof(a));
  a.src = src;
  a.tb = tb;
  a.w = w;
  a.scales = scales;
  a.nproj = nproj;
  a.chunk_begin[0] = 0;
  for (int p = 0; p < nproj; ++p) {
    if (!y[p] || !delta[p]) return fail(SLORA_ERR_NULL, "y[%d] or delta[%d] is null", p, p);
    if (qkvo[p] < 0 || qkvo[p] > 3) return fail(SLORA_ERR_QKVO, "qkvo=%d outside 0..3", qkvo[p]);
    if (h_out[p] <= 0 || h_out[p] % 8 != 0 || h_out[p] >= 65536 * 8)
      return fail(SLORA_ERR_SHAPE, "No suitable kernel. h_out=%d must be a positive multiple of 8", h_out[p]);
    a.y[p] = y[p];
    a.y_stride[p] = y_stride[p];
    a.h_out[p] = h_out[p];
    a.delta[p] = delta[p];
    a.qkvo[p] = qkvo[p];
    const int64_t chunks = (static_cast<int64_t>(h_out[p]) * max_rank + kChunk - 1) / kChunk;
    a.chunk_begin[p + 1] = a.chunk_begin[p] + static_cast<int>(chunks);
  }
  a.delta_stride = delta_stride;
  a.delta_parts = delta_parts;
  a.delta_part_stride = delta_part_stride;
  a.rank_mult = rank_mult;
  a.piece = piece;
  a.status = status;
  int slots = 0;
  tile_src_slots(src, tb.n_adapters, &slots);
  const int64_t grid = static_cast<int64_t>(slots) * a.chunk_begin[nproj];
  if (dtype == SLORA_F16) return launch(lora_expand_kernel<__half>, grid, 0, flags, stream, a, "expand");
  return launch(lora_expand_kernel<__nv_bfloat16>, grid, 0, flags, stream, a, "expand");
}

int make_src(const void* plan, const int64_t* ids, int64_t T, TileSrc* src, int32_t** status) {
  memset(src, 0, sizeof(*src));
  src->T = T;
  *status = nullptr;
  if (T < 0 || T > 0x3fffffff) return fail(SLORA_ERR_SHAPE, "T=%lld out of range", (long long)T);
  if (plan) {
    if (!aligned16(plan)) return fail(SLORA_ERR_ALIGN, "plan workspace is not 16-byte aligned");
    src->mode = MODE_PLAN;
    src->plan = reinterpret_cast<const int32_t*>(plan);
    *status = const_cast<int32_t*>(src->plan) + PH_STATUS;
  } else {
    if (!ids && T > 0) return fail(SLORA_ERR_NULL, "neither plan nor ids given");
    src->mode = MODE_TOKEN;
    src->ids = ids;
  }
  return SLORA_OK;
}

int make_seg_src(const int32_t* seg_start, const int32_t* seg_len, const int64_t* seg_adapter, int n_seg,
                 int max_seg_len, int64_t T, TileSrc* src) {
  memset(src, 0, sizeof(*src));
  if (n_seg < 0 || max_seg_len < 0 || T < 0) return fail(SLORA_ERR_SHAPE, "negative segment count or length");
  if (n_seg > 0 && (!seg_start || !seg_len || !seg_adapter)) return fail(SLORA_ERR_NULL, "null segment table");
  src->mode = MODE_SEGMENT;
  src->ids = seg_adapter;
  src->seg_start = seg_start;
  src->seg_len = seg_len;
  src->n_seg = n_seg;
  src->tiles_per_seg = (max_seg_len + kTileTokens - 1) / kTileTokens;
  src->T = (n_seg == 0 || src->tiles_per_seg == 0) ? 0 : T;
  return SLORA_OK;
}

Tables make_tables(const int64_t* start, const int64_t* ranks4, const int64_t* loc, int64_t n_adapters,
                   int64_t loc_len, int64_t pool_rows, int64_t pool_stride) {
  Tables tb;
  tb.start = start;
  tb.ranks4 = ranks4;
  tb.loc = loc;
  tb.n_adapters = n_adapters;
  tb.loc_len = loc_len;
  tb.pool_rows = pool_rows;
  tb.pool_stride = pool_stride;
  return tb;
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------------------
extern "C" {

int slora_version(void) { return 100; }

const char* slora_last_error(void) { return g_err; }

int slora_bgmv_shrink(void* delta, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int64_t* ids, int qkvo, int64_t T, int h_in, int64_t x_stride,
                      int64_t delta_stride, int delta_width, int64_t pool_rows, int64_t pool_stride,
                      int64_t n_adapters, int64_t loc_len, int dtype, void* stream) {
  TileSrc src;
  int32_t* status;
  int rc = make_src(nullptr, ids, T, &src, &status);
  if (rc) return rc;
  void* d[1] = {delta};
  const int q[1] = {qkvo};
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), w, x,
                    x_stride, h_in, 1, q, d, delta_stride, delta_width, dtype, 0, nullptr,
                    static_cast<cudaStream_t>(stream));
}

int slora_bgmv_expand(void* y, const void* delta, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int64_t* ids, const void* scales, int qkvo, int64_t T, int h_out,
                      int64_t delta_stride, int delta_width, int64_t y_stride, int64_t pool_rows,
                      int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype, void* stream) {
  TileSrc src;
  int32_t* status;
  int rc = make_src(nullptr, ids, T, &src, &status);
  if (rc) return rc;
  void* yy[1] = {y};
  const void* d[1] = {delta};
  const int q[1] = {qkvo};
  const int64_t ys[1] = {y_stride};
  const int ho[1] = {h_out};
  return run_expand(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), w, scales, 1,
                    q, yy, ys, ho, d, delta_stride, delta_width, 1, 0, 1, dtype, 0, nullptr,
                    static_cast<cudaStream_t>(stream));
}

int slora_dispatch_bgmv(void* y, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                        const int64_t* loc, const int64_t* ids, int qkvo, const void* scales, int64_t T, int h_in,
                        int h_out, int64_t pool_rows, int64_t pool_stride, int64_t n_adapters, int64_t loc_len,
                        int dtype, void* stream) {
  if (T == 0) return SLORA_OK;
  if (!y || !x) return fail(SLORA_ERR_NULL, "x or y is null");
  if (h_in < h_out) {
    return slora_bgmv_expand(y, x, w, start, ranks4, loc, ids, scales, qkvo, T, h_out, h_in, h_in, h_out,
                             pool_rows, pool_stride, n_adapters, loc_len, dtype, stream);
  }
  return slora_bgmv_shrink(y, x, w, start, ranks4, loc, ids, qkvo, T, h_in, h_in, h_out, h_out, pool_rows,
                           pool_stride, n_adapters, loc_len, dtype, stream);
}

int slora_sgmv_shrink(void* delta, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int32_t* seg_start, const int32_t* seg_len,
                      const int64_t* seg_adapter, int n_seg, int max_seg_len, int qkvo, int64_t T, int h_in,
                      int64_t x_stride, int64_t delta_stride, int delta_width, int64_t pool_rows,
                      int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype, void* stream) {
  TileSrc src;
  int rc = make_seg_src(seg_start, seg_len, seg_adapter, n_seg, max_seg_len, T, &src);
  if (rc) return rc;
  void* d[1] = {delta};
  const int q[1] = {qkvo};
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), w, x,
                    x_stride, h_in, 1, q, d, delta_stride, delta_width, dtype, 0, nullptr,
                    static_cast<cudaStream_t>(stream));
}

int slora_sgmv_expand(void* y, const void* delta, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int32_t* seg_start, const int32_t* seg_len,
                      const int64_t* seg_adapter, const void* scales, int n_seg, int max_seg_len, int qkvo,
                      int64_t T, int h_out, int64_t delta_stride, int delta_width, int64_t y_stride,
                      int64_t pool_rows, int64_t pool_stride, int64_t n_adapters, int64_t loc_len, int dtype,
                      void* stream) {
  TileSrc src;
  int rc = make_seg_src(seg_start, seg_len, seg_adapter, n_seg, max_seg_len, T, &src);
  if (rc) return rc;
  void* yy[1] = {y};
  const void* d[1] = {delta};
  const int q[1] = {qkvo};
  const int64_t ys[1] = {y_stride};
  const int ho[1] = {h_out};
  return run_expand(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), w, scales, 1,
                    q, yy, ys, ho, d, delta_stride, delta_width, 1, 0, 1, dtype, 0, nullptr,
                    static_cast<cudaStream_t>(stream));
}

size_t slora_plan_workspace_bytes(int64_t T, int64_t n_adapters) {
  if (T < 0 || n_adapters < 0) return 0;
  return plan_layout(T, n_adapters).words * sizeof(int32_t);
}

int slora_plan_build(void* workspace, size_t workspace_bytes, const int64_t* ids, int64_t T, int64_t n_adapters,
                     void* stream) {
  if (!workspace || (!ids && T > 0)) return fail(SLORA_ERR_NULL, "workspace or ids is null");
  if (!aligned16(workspace)) return fail(SLORA_ERR_ALIGN, "plan workspace is not 16-byte aligned");
  if (T < 0 || T > 0x3fffffff || n_adapters < 0 || n_adapters > 0x3fffffff)
    return fail(SLORA_ERR_SHAPE, "T=%lld or n_adapters=%lld out of range", (long long)T, (long long)n_adapters);
  const PlanLayout l = plan_layout(T, n_adapters);
  if (workspace_bytes < l.words * sizeof(int32_t))
    return fail(SLORA_ERR_WORKSPACE, "plan workspace has %zu bytes, needs %zu", workspace_bytes,
                l.words * sizeof(int32_t));
  plan_build_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<int32_t*>(workspace), ids, static_cast<int>(T), static_cast<int>(n_adapters), l.max_tiles);
  plan_fence_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
  return check_launch("plan_build");
}

int slora_plan_status(const void* workspace, int* status_out, int* n_tiles_out, void* stream) {
  if (!workspace) return fail(SLORA_ERR_NULL, "workspace is null");
  int32_t hdr[PH_WORDS];
  cudaError_t e = cudaMemcpyAsync(hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "plan_status: %s", cudaGetErrorString(e));
  if (hdr[PH_MAGIC] != kPlanMagic) return fail(SLORA_ERR_WORKSPACE, "workspace does not hold a plan");
  if (status_out) *status_out = hdr[PH_STATUS];
  if (n_tiles_out) *n_tiles_out = hdr[PH_NTILES];
  return SLORA_OK;
}

int slora_lora_shrink_multi(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* delta,
                            int64_t delta_stride, int delta_width, const void* x, int64_t x_stride, int h_in,
                            const void* pool_a, int64_t pool_rows, int64_t pool_stride, const int64_t* start,
                            const int64_t* ranks4, const int64_t* loc, int64_t n_adapters, int64_t loc_len,
                            int64_t T, int dtype, unsigned flags, void* stream) {
  if (!qkvo || !delta) return fail(SLORA_ERR_NULL, "qkvo or delta array is null");
  TileSrc src;
  int32_t* status;
  int rc = make_src(plan, ids, T, &src, &status);
  if (rc) return rc;
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_a, x,
                    x_stride, h_in, nproj, qkvo, delta, delta_stride, delta_width, dtype, flags, status,
                    static_cast<cudaStream_t>(stream));
}

int slora_lora_expand_multi(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* y,
                            const int64_t* y_stride, const int* h_out, const void* const* delta,
                            int64_t delta_stride, int delta_width, int delta_parts, int64_t delta_part_stride,
                            int rank_mult, const void* pool_b, int64_t pool_rows, int64_t pool_stride,
                            const int64_t* start, const int64_t* ranks4, const int64_t* loc, const void* scales,
                            int64_t n_adapters, int64_t loc_len, int64_t T, int dtype, unsigned flags,
                            void* stream) {
  if (!qkvo || !y || !y_stride || !h_out || !delta) return fail(SLORA_ERR_NULL, "null argument array");
  TileSrc src;
  int32_t* status;
  int rc = make_src(plan, ids, T, &src, &status);
  if (rc) return rc;
  return run_expand(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_b,
                    scales, nproj, qkvo, y, y_stride, h_out, delta, delta_stride, delta_width, delta_parts,
                    delta_part_stride, rank_mult, dtype, flags, status, static_cast<cudaStream_t>(stream));
}

int slora_batch_lora_qkv(const void* plan, const int64_t* ids, void* q, void* k, void* v, int64_t q_stride,
                         int64_t k_stride, int64_t v_stride, int h_out_q, int h_out_kv, const void* x,
                         int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         const void* scales, int64_t n_adapters, int64_t loc_len, void* delta_q, void* delta_k,
                         void* delta_v, int64_t delta_stride, int delta_width, int64_t T, int dtype,
                         unsigned flags, void* stream) {
  const int qkvo[3] = {0, 1, 2};
  void* d[3] = {delta_q, delta_k, delta_v};
  int rc = slora_lora_shrink_multi(plan, ids, 3, qkvo, d, delta_stride, delta_width, x, x_stride, h_in, pool_a,
                                   pool_rows, pool_stride, start, ranks4, loc, n_adapters, loc_len, T, dtype, flags,
                                   stream);
  if (rc) return rc;
  void* y[3] = {q, k, v};
  const int64_t ys[3] = {q_stride, k_stride, v_stride};
  const int ho[3] = {h_out_q, h_out_kv, h_out_kv};
  const void* dc[3] = {delta_q, delta_k, delta_v};
  return slora_lora_expand_multi(plan, ids, 3, qkvo, y, ys, ho, dc, delta_stride, delta_width, 1, 0, 1, pool_b,
                                 pool_rows, pool_stride, start, ranks4, loc, scales, n_adapters, loc_len, T, dtype,
                                 flags, stream);
}

int slora_batch_lora_o(const void* plan, const int64_t* ids, void* o, int64_t o_stride, int h_out, const void* x,
                       int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                       int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                       const void* scales, int64_t n_adapters, int64_t loc_len, void* delta, int64_t delta_stride,
                       int delta_width, int64_t T, int dtype, unsigned flags, void* stream) {
  const int qkvo[1] = {3};
  void* d[1] = {delta};
  int rc = slora_lora_shrink_multi(plan, ids, 1, qkvo, d, delta_stride, delta_width, x, x_stride, h_in, pool_a,
                                   pool_rows, pool_stride, start, ranks4, loc, n_adapters, loc_len, T, dtype, flags,
                                   stream);
  if (rc) return rc;
  void* y[1] = {o};
  const int64_t ys[1] = {o_stride};
  const int ho[1] = {h_out};
  const void* dc[1] = {delta};
  return slora_lora_expand_multi(plan, ids, 1, qkvo, y, ys, ho, dc, delta_stride, delta_width, 1, 0, 1, pool_b,
                                 pool_rows, pool_stride, start, ranks4, loc, scales, n_adapters, loc_len, T, dtype,
                                 flags, stream);
}

int slora_validate_tables(const int64_t* start, const int64_t* ranks4, const int64_t* loc, const int64_t* ids,
                          int64_t n_adapters, int64_t loc_len, int64_t T, int64_t pool_rows, int32_t* report,
                          void* stream) {
  if (!start || !ranks4 || !loc || !report) return fail(SLORA_ERR_NULL, "null table or report pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  zero_report_kernel<<<1, 32, 0, s>>>(report);
  validate_tables_kernel<<<64, 256, 0, s>>>(start, ranks4, loc, ids, n_adapters, loc_len, T, pool_rows, report);
  return check_launch("validate_tables");
}

}  // extern "C"
