// Shrink and expand of one call in ONE persistent launch (same-rank decode batches).
//
// The two-launch path pays the fixed part of a launch twice per call (launch, table chase, first bulk copy, drain),
// and the expand cannot read a delta row before the whole shrink grid has retired.  For a decode batch of small-rank
// adapters those fixed parts are as long as the streaming itself.  Here the unit of work is (tile, projection): the
// CTA that owns a unit runs its shrink row blocks and then its expand chunks back to back through one ring, so
//   * the adapter rows of A and of B stream without a gap (B chunks are on their way while the shrink computes),
//   * the intermediate never leaves the SM: the shrink's last-arriving consumer warp rounds it to the I/O type (as
//     the two-launch path does when it stores delta) and leaves it in shared memory for the expand stages,
//   * no CTA waits for another CTA.
// Work items, stage layouts and the arithmetic are those of lora_shrink_pipe_kernel / lora_expand_pipe_kernel
// (padded enumeration), so the results are bit-identical to the two-launch path.
//
// Order inside a CTA: units u = blockIdx.x + k * gridDim.x; per unit first its max_rb shrink items (row blocks of
// kMaxRows rows), then its expand chunks.  Consumer warps take stages in ring order; an expand stage carries the
// number of shrink items issued before it and waits (bounded) until that many have been completed - by then the
// warp itself has finished its part of them, it only waits for the slowest sibling warp.
#pragma once

#include "lora_pipelined.cuh"

namespace slora {

constexpr int kFusedRingBytes = 92 * 1024;  // ring + control blocks of two CTAs fit one SM
constexpr int FLAG_EXPAND = 8;              // stage kind (stage meta word 0; the shrink-item count sits above bit 8)
constexpr int FLAG_ZERO = 16;               // shrink item whose table entries were bad: its delta rows become zero
constexpr int kFusedDeltaStride = 128 + 8;  // elements per token row of the shared-memory intermediate

struct FusedArgs {
  ShrinkArgs s;  // src, tables, A pool, x; delta pointers unused
  ExpandArgs e;  // B pool, scales, y
  int e_max;     // chunks of the projection with the most chunks
  int ipu;       // items enumerated per unit = s.max_rb + e_max
};

struct FusedCtl {
  ShrinkRed red;
  int s_done;  // shrink items completed by this CTA so far
  __align__(16) unsigned short delta[kTileTokens][kFusedDeltaStride];
};

template <typename T>
__device__ __forceinline__ void fused_producer(const FusedArgs& a, unsigned char* ring_mem, PipeCtl& c, int lane) {
  const ShrinkArgs& sa = a.s;
  const ExpandArgs& ea = a.e;
  const int h_in = sa.h_in;
  const int64_t S = sa.tb.pool_stride;
  const T* wa = reinterpret_cast<const T*>(sa.w);
  const T* wb = reinterpret_cast<const T*>(ea.w);
  const T* x = reinterpret_cast<const T*>(sa.x);
  const int64_t G = gridDim.x;
  const uint32_t ring_base = smem_u32(ring_mem);
  PipeCtl::Prod& pp = c.prod[0];
  Ring r;
  r.cap = kFusedRingBytes;
  r.status = sa.status;
  const int nproj = sa.nproj;
  const int64_t n_units = static_cast<int64_t>(tile_count(sa.src)) * nproj;
  const int64_t my_units = n_units > blockIdx.x ? (n_units - blockIdx.x + G - 1) / G : 0;
  const int64_t n_local = my_units * a.ipu;
  int s_issued = 0;  // shrink items issued so far (the same in every lane)

  for (int64_t q0 = 0; q0 < n_local && !r.dead; q0 += 32) {
    // ---- 32 items resolved in parallel, one per lane ----
    // kind: 0 nothing, 1 shrink item, 2 expand item, 3 shrink item that only zeroes its delta rows
    // shrink: d_i = {-, n, nrows, j0, p, r, -, -, tok[8]}, d_l[j] = element offset of adapter row j
    // expand: d_i = {pr0, n, rk, p, clen, first output, scale bits, c0, tok[8]}, d_l[j] = pool row of slot row pr0 + j
    const int64_t q = q0 + lane;
    int kind = 0;
    if (q < n_local) {
      const int64_t k = q / a.ipu;
      const int j = static_cast<int>(q - k * a.ipu);
      const int64_t u = blockIdx.x + k * G;
      const int tile = static_cast<int>(u / nproj);
      const int p = static_cast<int>(u - static_cast<int64_t>(tile) * nproj);
      TileInfo t;
      if (lookup_tile(sa.src, sa.tb, tile, t, sa.status)) {
        const int64_t base = t.loc_base + static_cast<int64_t>(t.r) * pick3(sa.qkvo, p);
        if (j < sa.max_rb) {
          const int j0 = j * kMaxRows;
          const int rows_total = shrink_rows_of(sa, t.r);
          if (j0 < rows_total) {
            const int nrows = min(kMaxRows, rows_total - j0);
            bool ok = true;
#pragma unroll
            for (int jj = 0; jj < kMaxRows; ++jj) {
              if (jj < nrows) {
                const int64_t f = static_cast<int64_t>(j0 + jj) * h_in;
                const int64_t pr = f / S, col = f - pr * S;
                const int64_t e = pr < t.r ? sa.tb.loc[base + pr] : -1;
                if (e < 0 || e >= sa.tb.pool_rows) ok = false;
                pp.d_l[lane][jj] = e * S + col;
              }
            }
#pragma unroll
            for (int i = 0; i < kTileTokens; ++i) pp.d_i[lane][8 + i] = i < t.n ? tile_token(t, i) : 0;
            pp.d_i[lane][1] = t.n;
            pp.d_i[lane][2] = nrows;
            pp.d_i[lane][3] = j0;
            pp.d_i[lane][4] = p;
            pp.d_i[lane][5] = t.r;
            kind = ok ? 1 : 3;
            if (!ok) set_status(sa.status, SLORA_STATUS_BAD_TABLE);
          }
        } else {
          const int ch = j - sa.max_rb;
          const int rk = t.r * ea.rank_mult;
          if (!expand_rank_ok(ea, rk)) {
            if (ch == 0) set_status(ea.status, SLORA_STATUS_BAD_RANK);
          } else if (ch < expand_chunks_of(ea, p, rk)) {
            const int h_out = pick3(ea.h_out, p);
            const int64_t flat_total = static_cast<int64_t>(h_out) * rk;
            const int64_t c0 = static_cast<int64_t>(ch) * kPipeChunk;
            if (c0 < flat_total) {
              const int clen = static_cast<int>(min(static_cast<int64_t>(kPipeChunk), flat_total - c0));
              const int64_t pr0 = c0 / S, pr1 = (c0 + clen - 1) / S;
              bool ok = pr1 - pr0 < kSpanRows && pr1 < t.r;
              if (ok) {
#pragma unroll
                for (int jj = 0; jj < kSpanRows; ++jj) {
                  if (pr0 + jj <= pr1) {
                    const int64_t e = ea.tb.loc[base + pr0 + jj];
                    if (e < 0 || e >= ea.tb.pool_rows) ok = false;
                    pp.d_l[lane][jj] = e;
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
                pp.d_i[lane][6] = __float_as_int(to_f32<T>(reinterpret_cast<const T*>(ea.scales)[t.adapter]));
                pp.d_i[lane][7] = static_cast<int>(c0);
                kind = 2;
              } else {
                set_status(ea.status, SLORA_STATUS_BAD_TABLE);
              }
            }
          }
        }
      }
    }
    const uint32_t any_mask = __ballot_sync(FULL_MASK, kind != 0);
    const uint32_t e_mask = __ballot_sync(FULL_MASK, kind == 2);
    const uint32_t z_mask = __ballot_sync(FULL_MASK, kind == 3);
    __syncwarp();

    // ---- feed the ring, item by item, in enumeration order ----
    for (uint32_t left = any_mask; left != 0 && !r.dead; left &= left - 1) {
      const int k = __ffs(left) - 1;
      const int* di = pp.d_i[k];
      if (!((e_mask >> k) & 1u)) {
        // shrink item: lane j < kMaxRows carries adapter row j, lane kMaxRows + i carries token i
        const bool zero = (z_mask >> k) & 1u;
        const int n = di[1], nrows = di[2];
        const bool is_w = !zero && lane < nrows;
        const bool is_x = !zero && lane >= kMaxRows && lane < kMaxRows + n;
        const int mytok = (lane >= kMaxRows && lane < kMaxRows + kTileTokens) ? di[8 + lane - kMaxRows] : 0;
        const T* src0 = is_w ? wa + pp.d_l[k][lane & (kMaxRows - 1)] : x + static_cast<int64_t>(mytok) * sa.x_stride;
        const int myslot = is_w ? lane : nrows + (lane - kMaxRows);
        const int fit = kMaxStageBytes / ((nrows + n) * static_cast<int>(sizeof(T))) / 2048 * 2048;
        const int kc_elems = zero ? h_in : (fit < 2048 ? 2048 : fit);  // same K-chunks as the two-launch shrink
        for (int k0 = 0; k0 < h_in; k0 += kc_elems) {
          const int klen = min(kc_elems, h_in - k0);
          const uint32_t bytes = static_cast<uint32_t>(klen) * sizeof(T);
          const uint32_t sz = zero ? 0u : round128(static_cast<uint32_t>(nrows + n) * bytes);
          const uint32_t off = ring_alloc(r, c, sz, lane);
          if (r.dead) break;
          const uint32_t slot = r.g % kSlots;
          r.head = off + sz;
          if (lane == 0) {
            pp.off[slot] = off;
            c.meta[slot][0] = (k0 == 0 ? FLAG_FIRST : 0) | (k0 + klen >= h_in ? FLAG_LAST : 0) | (zero ? FLAG_ZERO : 0);
            c.meta[slot][1] = nrows;
            c.meta[slot][2] = n;
            c.meta[slot][3] = di[3];
            c.meta[slot][4] = di[4];
            c.meta[slot][5] = klen;
            c.meta[slot][6] = static_cast<int>(off);
            c.meta[slot][7] = di[5];
          } else if (lane >= kMaxRows && lane < kMaxRows + kTileTokens) {
            c.meta[slot][8 + lane - kMaxRows] = mytok;
          }
          __syncwarp();
          if (lane == 0) mbar_expect_tx(&c.full[slot], zero ? 0u : static_cast<uint32_t>(nrows + n) * bytes);
          ring_issue(r, c, slot, ring_base + off + static_cast<uint32_t>(myslot) * bytes, src0 + k0,
                     (is_w || is_x) ? bytes : 0u, is_x, lane);
        }
        ++s_issued;
      } else {
        // expand item: lanes 0..15 carry pieces of the B chunk, lanes 16..23 the tokens' y segments
        const int n = di[1], rk = di[2], p = di[3], clen = di[4], obase = di[5];
        const int nout = clen / rk;
        const uint32_t b_bytes = static_cast<uint32_t>(clen) * sizeof(T);
        const uint32_t y_bytes = static_cast<uint32_t>(nout) * sizeof(T);
        const uint32_t total = b_bytes + static_cast<uint32_t>(n) * y_bytes;
        const uint32_t sz = round128(total);
        const uint32_t off = ring_alloc(r, c, sz, lane);
        if (r.dead) break;
        const uint32_t slot = r.g % kSlots;
        r.head = off + sz;
        const int mytok = lane >= 16 ? di[8 + (lane & 7)] : 0;
        if (lane == 0) {
          pp.off[slot] = off;
          c.meta[slot][0] = FLAG_EXPAND | (s_issued << 8);
          c.meta[slot][1] = n;
          c.meta[slot][2] = rk;
          c.meta[slot][3] = p;
          c.meta[slot][4] = clen;
          c.meta[slot][5] = obase;
          c.meta[slot][6] = di[6];
          c.meta[slot][7] = static_cast<int>(off);
        } else if (lane >= 16 && lane < 24) {
          c.meta[slot][8 + lane - 16] = mytok;
        }
        uint32_t dst = ring_base + off, bytes = 0;
        const T* src = wb;
        bool is_act = false;
        if (lane < kMaxPieces) {
          const int poff = lane * ea.piece;
          if (poff < clen) {
            const int64_t f = static_cast<int64_t>(di[7]) + poff;
            const int64_t pr = f / S, col = f - pr * S;
            src = wb + pp.d_l[k][static_cast<int>(pr) - di[0]] * S + col;
            dst += static_cast<uint32_t>(poff) * sizeof(T);
            bytes = static_cast<uint32_t>(min(ea.piece, clen - poff)) * sizeof(T);
          }
        } else if (lane < 16 + n) {
          src = reinterpret_cast<const T*>(pick3(ea.y, p)) + static_cast<int64_t>(mytok) * pick3(ea.y_stride, p) + obase;
          dst += b_bytes + static_cast<uint32_t>(lane - 16) * y_bytes;
          bytes = y_bytes;
          is_act = true;
        }
        __syncwarp();
        if (lane == 0) mbar_expect_tx(&c.full[slot], total);
        ring_issue(r, c, slot, dst, src, bytes, is_act, lane);
      }
    }
    __syncwarp();
  }
  ring_finish(r, c, sa.status, lane);
}

template <typename T>
__device__ __forceinline__ void fused_consumer(const FusedArgs& a, const unsigned char* ring_mem, PipeCtl& c,
                                               FusedCtl& f, int lane, int cw) {
  pdl_wait();
  float acc[kMaxRows][kTileTokens];
#pragma unroll
  for (int j = 0; j < kMaxRows; ++j) {
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) acc[j][i] = 0.f;
  }
  uint32_t item_seq = 0;
  const T* delta_s = reinterpret_cast<const T*>(&f.delta[0][0]);
  for (uint32_t g = 0;; ++g) {
    const uint32_t slot = g % kSlots;
    if (!mbar_wait_timed(&c.full[slot], (g / kSlots) & 1)) {
      if (lane == 0) set_status(a.s.status, SLORA_STATUS_TIMEOUT);
      return;
    }
    const int* m = c.meta[slot];
    const int flags = m[0];
    if (flags & FLAG_END) return;
    if (flags & FLAG_EXPAND) {
      // the unit's shrink items must all be complete (this warp's part of them is; wait for the slowest sibling)
      const int need = flags >> 8;
      const volatile int* done = &f.s_done;
      if (*done < need) {
        const long long t0 = clock64();
        while (*done < need) {
          if (clock64() - t0 > kWaitCycles) {
            if (lane == 0) set_status(a.e.status, SLORA_STATUS_TIMEOUT);
            return;
          }
        }
      }
      __threadfence_block();
      const T* bs = reinterpret_cast<const T*>(ring_mem + m[7]);
      const int p = m[3];
      T* y = reinterpret_cast<T*>(pick3(a.e.y, p));
      const int64_t ystr = pick3(a.e.y_stride, p);
      if (m[4] == kPipeChunk) {
        switch (m[2]) {
          case 8: expand_stage<T, 1, true>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 16: expand_stage<T, 2, true>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 32: expand_stage<T, 4, true>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 64: expand_stage<T, 8, true>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          default: expand_stage<T, 16, true>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
        }
      } else {
        switch (m[2]) {
          case 8: expand_stage<T, 1, false>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 16: expand_stage<T, 2, false>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 32: expand_stage<T, 4, false>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          case 64: expand_stage<T, 8, false>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
          default: expand_stage<T, 16, false>(bs, m, y, ystr, lane, cw, delta_s, kFusedDeltaStride); break;
        }
      }
    } else {
      const int nrows = m[1], n = m[2], klen = m[5];
      if (flags & FLAG_FIRST) {
#pragma unroll
        for (int j = 0; j < kMaxRows; ++j) {
#pragma unroll
          for (int i = 0; i < kTileTokens; ++i) acc[j][i] = 0.f;
        }
      }
      if (!(flags & FLAG_ZERO)) {
        const T* st = reinterpret_cast<const T*>(ring_mem + m[6]);
        if (n <= 1) {
          shrink_accumulate<T, 1>(acc, st, nrows, n, klen, cw, lane);
        } else if (n <= 2) {
          shrink_accumulate<T, 2>(acc, st, nrows, n, klen, cw, lane);
        } else if (n <= 4) {
          shrink_accumulate<T, 4>(acc, st, nrows, n, klen, cw, lane);
        } else {
          shrink_accumulate<T, 8>(acc, st, nrows, n, klen, cw, lane);
        }
      }
      if (flags & FLAG_LAST) {
        const uint32_t buf = item_seq % kSlots;
        ++item_seq;
        float* red_row = f.red.sum[buf][cw];
        int nt;
        if (n <= 1) {
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
          old = atomicAdd(&f.red.cnt[buf], 1);
        }
        old = __shfl_sync(FULL_MASK, old, 0);
        if (old == kConsumerWarps - 1) {
          __threadfence_block();
          const int j = lane / nt, i = lane - j * nt;
          if (lane < kMaxRows * nt) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) sum += f.red.sum[buf][w][lane];
            if (j < nrows && i < n && m[3] + j < a.s.delta_width && m[3] + j < kFusedDeltaStride) {
              // rounded to the I/O type exactly where the two-launch path rounds it (its store of delta)
              reinterpret_cast<T*>(&f.delta[i][0])[m[3] + j] = from_f32<T>(sum);
            }
          }
          __syncwarp();
          if (lane == 0) {
            f.red.cnt[buf] = 0;
            __threadfence_block();
            atomicAdd(&f.s_done, 1);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPipeThreads, kPipeCtasPerSm) lora_fused_pipe_kernel(const FusedArgs a) {
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(16) PipeCtl ctl;
  __shared__ __align__(16) FusedCtl fctl;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < kSlots) fctl.red.cnt[tid] = 0;
  if (tid == 0) fctl.s_done = 0;
  pipe_init(ctl, tid);
  pdl_launch_dependents();
  if (warp < kProducerWarps) {
    fused_producer<T>(a, ring_mem, ctl, lane);
  } else {
    fused_consumer<T>(a, ring_mem, ctl, fctl, lane, warp - kProducerWarps);
  }
}

}  // namespace slora
