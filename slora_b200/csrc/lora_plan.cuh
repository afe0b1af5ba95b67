// Batch plan: group the tokens of one batch by adapter (one CTA; T and n_adapters are a few thousand at most).
#pragma once

#include "lora_common.cuh"

namespace slora {

// workspace words: [header PH_WORDS][tile records kTileWords * max_tiles][perm T][pos T][cnt n_adapters]
//                  [big-tile records kTileWords * max_big][resolved tiles (kXtHead + 4 * xrcap) * max_tiles, optional]
// Counting sort by adapter id: histogram, exclusive scan over adapters (tokens and tiles at once), scatter.
// Tokens whose id is outside [0, n_adapters) are left out and SLORA_STATUS_BAD_ID is recorded; adapters whose
// table entries are out of range get tiles of zero tokens and SLORA_STATUS_BAD_TABLE.
__global__ void __launch_bounds__(1024) plan_build_kernel(int32_t* ws, const int64_t* __restrict__ ids,
                                                          const int64_t* __restrict__ start,
                                                          const int64_t* __restrict__ ranks4, int64_t loc_len, int T,
                                                          int n_adapters, int max_tiles, int max_big,
                                                          const int64_t* __restrict__ loc,
                                                          const unsigned short* __restrict__ scales16, int xoff,
                                                          int xrcap) {
  int32_t* hdr = ws;
  int32_t* tiles = ws + PH_WORDS;
  int32_t* perm = tiles + kTileWords * max_tiles;
  int32_t* pos = perm + T;
  int32_t* cnt = pos + T;
  const int big_off = (PH_WORDS + kTileWords * max_tiles + 2 * T + n_adapters + 3) & ~3;  // 16-byte aligned records
  int32_t* big = ws + big_off;
  __shared__ int s_tok[32], s_tile[32], s_big[32];
  __shared__ int s_status, s_rmin, s_rmax, s_nsmall, s_big_rmax, s_big_pow2;
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < n_adapters; i += nthr) cnt[i] = 0;
  if (tid == 0) {
    s_status = 0;
    s_rmin = 0x7fffffff;
    s_rmax = 0;
    s_nsmall = 0;
    s_big_rmax = 0;
    s_big_pow2 = 1;
  }
  __syncthreads();
  for (int t = tid; t < T; t += nthr) {
    const int64_t a = ids[t];
    if (a < 0 || a >= n_adapters) {
      pos[t] = -1;
      atomicOr(&s_status, SLORA_STATUS_BAD_ID);
    } else {
      pos[t] = atomicAdd(&cnt[a], 1);
    }
  }
  __syncthreads();
  // exclusive scan over adapters of (tokens, tiles); each thread owns a contiguous run of adapters
  const int per = (n_adapters + nthr - 1) / nthr;
  const int lo = min(tid * per, n_adapters), hi = min(lo + per, n_adapters);
  // a group is big when it has kBigGroupTokens tokens or more and a rank the tensor-core kernels take
  auto is_big = [&](int a, int c) {
    if (c < kBigGroupTokens) return false;
    const int64_t r = ranks4[a] >> 2;
    return r >= 8 && r <= 128 && r % 8 == 0;
  };
  int tok_sum = 0, tile_sum = 0, big_sum = 0;
  for (int a = lo; a < hi; ++a) {
    const int c = cnt[a];
    tok_sum += c;
    tile_sum += (c + kTileTokens - 1) / kTileTokens;
    if (is_big(a, c)) big_sum += (c + kBigTileTokens - 1) / kBigTileTokens;
  }
  int tok_inc = tok_sum, tile_inc = tile_sum, big_inc = big_sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, tok_inc, off);
    const int b = __shfl_up_sync(0xffffffffu, tile_inc, off);
    const int g = __shfl_up_sync(0xffffffffu, big_inc, off);
    if (lane >= off) {
      tok_inc += a;
      tile_inc += b;
      big_inc += g;
    }
  }
  if (lane == 31) {
    s_tok[warp] = tok_inc;
    s_tile[warp] = tile_inc;
    s_big[warp] = big_inc;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = nthr >> 5;
    const int a = lane < nw ? s_tok[lane] : 0, b = lane < nw ? s_tile[lane] : 0, g = lane < nw ? s_big[lane] : 0;
    int ai = a, bi = b, gi = g;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a2 = __shfl_up_sync(0xffffffffu, ai, off);
      const int b2 = __shfl_up_sync(0xffffffffu, bi, off);
      const int g2 = __shfl_up_sync(0xffffffffu, gi, off);
      if (lane >= off) {
        ai += a2;
        bi += b2;
        gi += g2;
      }
    }
    s_tok[lane] = ai - a;  // exclusive
    s_tile[lane] = bi - b;
    s_big[lane] = gi - g;
    if (lane == 31) {
      hdr[PH_NTILES] = min(bi, max_tiles);
      hdr[PH_NBIG] = min(gi, max_big);
    }
  }
  __syncthreads();
  int tok_off = s_tok[warp] + tok_inc - tok_sum;
  int tile_off = s_tile[warp] + tile_inc - tile_sum;
  int bigt_off = s_big[warp] + big_inc - big_sum;
  for (int a = lo; a < hi; ++a) {
    const int c = cnt[a];
    cnt[a] = tok_off;  // becomes the group's first slot in perm
    if (c > 0) {
      const int64_t r4 = ranks4[a], st = start[a];
      const bool good = r4 >= 0 && st >= 0 && st + r4 <= loc_len && r4 <= (int64_t(1) << 20) && st < 0x7fffffffLL;
      if (!good) atomicOr(&s_status, SLORA_STATUS_BAD_TABLE);
      const bool bigg = good && is_big(a, c);
      if (good) {
        atomicMin(&s_rmin, static_cast<int>(r4 >> 2));
        atomicMax(&s_rmax, static_cast<int>(r4 >> 2));
      }
      if (bigg) {
        const int rr = static_cast<int>(r4 >> 2);
        atomicMax(&s_big_rmax, rr);
        if (rr & (rr - 1)) s_big_pow2 = 0;
      } else if (good) {
        atomicAdd(&s_nsmall, (c + kTileTokens - 1) / kTileTokens);
      }
      for (int i = 0; i * kTileTokens < c; ++i) {
        if (tile_off < max_tiles) {
          int4* rec = reinterpret_cast<int4*>(tiles + kTileWords * tile_off);
          rec[0] = make_int4(a, tok_off + i * kTileTokens, good ? min(kTileTokens, c - i * kTileTokens) : 0,
                             good ? static_cast<int>(r4 >> 2) : 0);
          rec[1] = make_int4(good ? static_cast<int>(st) : 0, bigg ? 1 : 0, 0, 0);
        }
        ++tile_off;
      }
      if (bigg) {
        for (int i = 0; i * kBigTileTokens < c; ++i) {
          if (bigt_off < max_big) {
            int4* rec = reinterpret_cast<int4*>(big + kTileWords * bigt_off);
            rec[0] = make_int4(a, tok_off + i * kBigTileTokens, min(kBigTileTokens, c - i * kBigTileTokens),
                               static_cast<int>(r4 >> 2));
            rec[1] = make_int4(static_cast<int>(st), 0, 0, 0);
          }
          ++bigt_off;
        }
      }
    }
    tok_off += c;
  }
  __syncthreads();
  for (int t = tid; t < T; t += nthr) {
    const int p = pos[t];
    if (p >= 0) perm[cnt[ids[t]] + p] = t;
  }
  // resolved tiles (see PH_XOFF): token ids, scale and pool rows of every tile whose rank the entries hold
  if (xoff > 0 && loc != nullptr) {
    __syncthreads();  // tile records and perm are complete
    const int ntiles = hdr[PH_NTILES];
    const int ew = kXtHead + 4 * xrcap;
    for (int tile = tid; tile < ntiles; tile += nthr) {
      int32_t* rec = tiles + kTileWords * tile;
      const int a = rec[0], first = rec[1], n = rec[2], r = rec[3];
      const bool filled = n > 0 && r > 0 && r <= xrcap;
      rec[6] = filled ? 1 : 0;
      if (filled) {
        int32_t* e = ws + xoff + static_cast<int64_t>(tile) * ew;
        for (int i = 0; i < kTileTokens; ++i) e[i] = i < n ? perm[first + i] : 0;
        e[8] = scales16 != nullptr ? (0x10000 | scales16[a]) : 0;
        e[9] = e[10] = e[11] = 0;
      }
    }
    // pool rows: one (tile, projection, row) per thread and step, four steps in flight (32-bit index arithmetic; the
    // table loads of a round are issued before any of them is used)
    const int per_tile = 4 * xrcap;
    const int total = ntiles * per_tile;  // at most a few hundred thousand
    for (int idx0 = tid; idx0 < total; idx0 += 4 * nthr) {
      int64_t v[4];
      int dst[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * nthr;
        dst[u] = -1;
        v[u] = -1;
        if (idx < total) {
          const int tile = idx / per_tile, q = idx - tile * per_tile;
          const int p = q / xrcap, j = q - p * xrcap;
          const int4 rec0 = *reinterpret_cast<const int4*>(tiles + kTileWords * tile);
          const int st = tiles[kTileWords * tile + 4];
          if (rec0.z > 0 && rec0.w > 0 && rec0.w <= xrcap && j < rec0.w) {
            v[u] = loc[static_cast<int64_t>(st) + static_cast<int64_t>(rec0.w) * p + j];
            dst[u] = xoff + tile * ew + kXtHead + p * xrcap + j;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (dst[u] >= 0) ws[dst[u]] = (v[u] >= 0 && v[u] < 0x7fffffffLL) ? static_cast<int32_t>(v[u]) : -1;
      }
    }
  }
  if (tid == 0) {
    hdr[PH_XOFF] = (xoff > 0 && loc != nullptr) ? xoff : 0;
    hdr[PH_XRCAP] = (xoff > 0 && loc != nullptr) ? xrcap : 0;
    hdr[PH_MAGIC] = kPlanMagic;
    hdr[PH_STATUS] = s_status;
    hdr[PH_MAXTILES] = max_tiles;
    hdr[PH_T] = T;
    hdr[PH_NADAPTERS] = n_adapters;
    hdr[PH_BIGOFF] = big_off;
    hdr[PH_MAXBIG] = max_big;
    hdr[PH_UNIFORM] = s_rmin == s_rmax ? s_rmax : 0;
    hdr[PH_NSMALL] = s_nsmall;
    hdr[PH_BIG_RMAX] = s_big_rmax;
    hdr[PH_BIG_POW2] = s_big_pow2;
  }
}

// Empty kernel launched (without programmatic serialization) right after plan_build_kernel: later kernels that
// start early under programmatic dependent launch read the plan before their grid-dependency wait, and this
// fully serialised launch in between guarantees the plan's writes are complete and visible by then.
__global__ void plan_fence_kernel() {}

}  // namespace slora
