// Simple (one CTA per work item) LoRA shrink / expand kernels.
//
// These serve every layout the library accepts (any pool stride that shares a 16-byte piece with the feature size,
// 2-byte aligned y, the all-gathered delta layout of tensor parallelism) and are the fallback of the pipelined
// kernels in lora_pipelined.cuh.  A CTA stages its adapter rows in shared memory with bulk asynchronous copies
// issued before the grid-dependency wait, then reduces (shrink) or expands (expand) them for the tile's tokens.
#pragma once

#include "lora_common.cuh"

namespace slora {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kTokPass = 4;                 // tokens reduced per register pass in the shrink
constexpr int kWarpSpan = kChunk / kWarps;  // 2048 flat elements per warp in the expand
constexpr int kShrinkSmemBudget = 64 * 1024;

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

  int32_t* status = a.status;
  TileInfo t;
  if (!lookup_tile(a.src, a.tb, tile_idx, t, tid == 0 ? status : nullptr)) return;
  const int r = t.r;
  const int64_t st = t.loc_base;
  const int j0 = rb * a.rows_per_cta;
  const int rows_total = r * a.rank_mult;  // A rows of the projection (rows may be shorter than a pool row)
  if (j0 >= rows_total) return;
  const int nrows = min(a.rows_per_cta, rows_total - j0);
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
  if (tid < t.n) s_tok[tid] = tile_token(t, tid);

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
  const int m_base = expand_m_base<LPO>(lane);
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
    expand_butterfly<LPO>(v, lane);
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

  int32_t* status = a.status;
  TileInfo t;
  if (!lookup_tile(a.src, a.tb, tile_idx, t, tid == 0 ? status : nullptr)) return;
  const int64_t st = t.loc_base;
  const int slot = t.r;
  const int r = slot * a.rank_mult;
  if (r == 0) return;
  const int h_out = a.h_out[p];
  const int64_t flat_total = static_cast<int64_t>(h_out) * r;
  const int64_t c0 = static_cast<int64_t>(c) * kChunk;
  if (c0 >= flat_total) return;
  if ((r != 8 && r != 16 && r != 32 && r != 64 && r != 128) || r > a.max_rank) {
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
  if (tid < t.n) s_tok[tid] = tile_token(t, tid);
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

}  // namespace slora
