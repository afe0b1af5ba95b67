// Expand with the two steps that follow it in the reference's layer folded into its epilogue: the rotary embedding of
// q and k (rotary_emb_fwd right after each expand, slora/models/peft/lora_unordered_batch_infer.py:277,298; kernel
// slora/models/llama/triton_kernel/rotary_emb.py:8-47) and the scatter of the new k and v rows into the KV pool
// (destindex_copy_kv, slora/common/basemodel/layer_infer/template/transformer_layer_infer_template.py:50-62; kernel
// slora/common/basemodel/triton_kernel/destindex_copy_kv.py:8-50).  The expand already has every output value in a
// register on its way to memory, so the rotation costs two more multiply-adds and the scatter only changes the row
// the value is written to: one pass over q, k and v instead of three (expand, rotary, copy).
//
// The rotary pairs elements d and d + 64 of a head (head_dim 128).  A consumer warp of the plain expand owns 2048
// consecutive flat B elements, i.e. 2048 / r consecutive outputs, which at rank 32 and more is less than a head:
// the two halves of a pair would sit in different warps.  Here the warp's eight 256-element loads are laid out
// pair-wise instead: loads 0..3 cover the low elements (d < 64) of the warp's pairs, loads 4..7 the high elements
// (d + 64) of the same pairs, so that after the butterfly (which hands lane l the outputs of loads m_base(l) + i) the
// partner of a value sits in the same lane (rank 8) or in lane l ^ 1 (all other ranks): one shuffle.
// Stage layout, work items and producer are those of lora_expand_pipe_kernel; only the consumer differs.
#pragma once

#include "lora_pipelined.cuh"

namespace slora {

constexpr int kRopeHeadDim = 128;

// What the epilogue needs beyond ExpandArgs.
struct RopeArgs {
  const void* cos;          // [T][64] in the I/O type: cosines of token t's position (infer_state.position_cos)
  const void* sin;
  int64_t cs_stride;        // elements between token rows of cos / sin
  int rope_mask;            // bit p: rotate the outputs of the call's projection p
  const int64_t* out_rows;  // when not null: row of out[p] that token t's result goes to (KV-pool row: dest index)
  void* out[3];             // out[p] null: projection p is updated in place in y[p]
  int64_t out_stride[3];
  int64_t out_rows_limit;   // rows of out[p]: a token whose out_rows entry is outside [0, limit) is skipped
};

template <typename T, int LPO, bool FULL, bool ROPE>
__device__ __forceinline__ void expand_stage_epi(const T* bs, const int* m, T* out_base, int64_t out_stride,
                                                 const int64_t* out_rows, int64_t out_rows_limit, const T* cosp,
                                                 const T* sinp, int64_t cs_stride, int lane, int cw, int32_t* status) {
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
  const int kp = (lane & (LPO - 1)) * 8;
  const int g = lane / LPO;
  // output (inside the chunk) that load mm brings this lane's 8 values of
  auto out_of = [&](int mm) {
    if (!ROPE) return (cw * 8 + mm) * OPL + g;
    const int pair = (cw * 4 + (mm & 3)) * OPL + g;  // pair index inside the chunk: 64 pairs per head
    return (pair >> 6) * kRopeHeadDim + (pair & 63) + (mm >> 2) * 64;
  };
  uint4 bv[8];
#pragma unroll
  for (int mm = 0; mm < 8; ++mm) {
    const int o = out_of(mm);
    bv[mm] = (FULL || o < nout) ? *reinterpret_cast<const uint4*>(bs + o * R + kp) : make_uint4(0u, 0u, 0u, 0u);
  }
  const int m_base = expand_m_base<LPO>(lane);
  const bool writer = (LPO < 16) || ((lane & 8) == 0);
  int o_loc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o_loc[i] = out_of(m_base + i);

  for (int tt = 0; tt < n; ++tt) {
    const uint4 dv = *reinterpret_cast<const uint4*>(ds + tt * R + kp);
    const int tok = m[8 + tt];
    float val[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      val[i] = (FULL || (writer && o_loc[i] < nout)) ? to_f32<T>(ys[tt * nout + o_loc[i]]) : 0.f;
    }
    float v[8];
#pragma unroll
    for (int mm = 0; mm < 8; ++mm) {
      v[mm] = 0.f;
      dot8<T>(v[mm], bv[mm], dv);
    }
    expand_butterfly<LPO>(v, lane);
    // y + scale * delta . B, rounded to the I/O type where the reference stores it before the rotary reads it back
#pragma unroll
    for (int i = 0; i < NV; ++i) val[i] = to_f32<T>(from_f32<T>(fmaf(scale, v[i], val[i])));
    if (ROPE) {
      float rot[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        // the other half of the pair: same lane, loads 4 apart (rank 8); else the neighbouring lane, same index
        const float other = LPO == 1 ? val[i ^ 4] : __shfl_xor_sync(FULL_MASK, val[i], 1);
        const bool high = LPO == 1 ? (i >= 4) : ((lane & 1) != 0);
        const int d = o_loc[i] & 63;
        const bool live = FULL || o_loc[i] < nout;
        const float c = live ? to_f32<T>(cosp[static_cast<int64_t>(tok) * cs_stride + d]) : 0.f;
        const float s = live ? to_f32<T>(sinp[static_cast<int64_t>(tok) * cs_stride + d]) : 0.f;
        // out0 = x0 cos - x1 sin;  out1 = x0 sin + x1 cos   (rotary_emb.py:39-40)
        rot[i] = high ? fmaf(other, s, val[i] * c) : fmaf(-other, s, val[i] * c);
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) val[i] = rot[i];
    }
    int64_t row = tok;
    if (out_rows != nullptr) {
      row = out_rows[tok];
      if (row < 0 || row >= out_rows_limit) {
        if (lane == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
        continue;  // (uniform over the warp: every lane looks at the same token)
      }
    }
    T* orow = out_base + row * out_stride + obase;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (writer && (FULL || o_loc[i] < nout)) orow[o_loc[i]] = from_f32<T>(val[i]);
    }
  }
}

template <typename T, bool ROPE>
__device__ __forceinline__ void expand_stage_epi_pick(const T* bs, const int* m, T* ob, int64_t os,
                                                      const int64_t* rows, int64_t limit, const T* cosp,
                                                      const T* sinp, int64_t css, int lane, int cw, int32_t* status) {
  if (m[4] == kPipeChunk) {
    switch (m[2]) {
      case 8: expand_stage_epi<T, 1, true, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 16: expand_stage_epi<T, 2, true, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 32: expand_stage_epi<T, 4, true, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 64: expand_stage_epi<T, 8, true, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      default: expand_stage_epi<T, 16, true, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
    }
  } else {
    switch (m[2]) {
      case 8: expand_stage_epi<T, 1, false, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 16: expand_stage_epi<T, 2, false, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 32: expand_stage_epi<T, 4, false, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      case 64: expand_stage_epi<T, 8, false, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
      default: expand_stage_epi<T, 16, false, ROPE>(bs, m, ob, os, rows, limit, cosp, sinp, css, lane, cw, status); break;
    }
  }
}

template <typename T>
__device__ __forceinline__ void expand_consumer_epi(const ExpandArgs& a, const RopeArgs& e,
                                                    const unsigned char* ring_mem, PipeCtl& c, int lane, int cw) {
  pdl_wait();
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
    void* redirect = pick3(e.out, p);
    T* ob = reinterpret_cast<T*>(redirect ? redirect : pick3(a.y, p));
    const int64_t os = redirect ? pick3(e.out_stride, p) : pick3(a.y_stride, p);
    const int64_t* rows = redirect ? e.out_rows : nullptr;
    const T* cosp = reinterpret_cast<const T*>(e.cos);
    const T* sinp = reinterpret_cast<const T*>(e.sin);
    if ((e.rope_mask >> p) & 1) {
      expand_stage_epi_pick<T, true>(bs, m, ob, os, rows, e.out_rows_limit, cosp, sinp, e.cs_stride, lane, cw, a.status);
    } else {
      expand_stage_epi_pick<T, false>(bs, m, ob, os, rows, e.out_rows_limit, cosp, sinp, e.cs_stride, lane, cw, a.status);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
}

template <typename T, bool EXACT>
__global__ void __launch_bounds__(kPipeThreads, kPipeCtasPerSm) lora_expand_rope_pipe_kernel(const ExpandArgs a, const RopeArgs e) {
  extern __shared__ __align__(128) unsigned char ring_mem[];
  __shared__ __align__(16) PipeCtl ctl;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pipe_init(ctl, tid);
  pdl_launch_dependents();
  if (EXACT) {
    fill_item_counts(a.src, a.tb, ctl, tid, [&](int rr, int) { return expand_items_of(a, rr); });
    __syncthreads();
  }
  if (warp < kProducerWarps) {
    expand_producer<T, EXACT>(a, ring_mem, ctl, lane, warp);
  } else {
    expand_consumer_epi<T>(a, e, ring_mem, ctl, lane, warp - kProducerWarps);
  }
}

// The same two steps as a pass of their own, for calls whose expand ran on another kernel family (tensor cores,
// simple kernels, head_dim other than 128): one CTA per (token, projection); rotation in FP32 from the stored values.
template <typename T>
__global__ void __launch_bounds__(128) rope_scatter_kernel(T* y0, T* y1, T* y2, int64_t s0, int64_t s1, int64_t s2,
                                                           int h0, int h1, int h2, int nproj, int head_dim,
                                                           const RopeArgs e, int32_t* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t tok = blockIdx.x;
  const int p = blockIdx.y;
  if (p >= nproj) return;
  T* y = p == 0 ? y0 : (p == 1 ? y1 : y2);
  const int64_t ys = p == 0 ? s0 : (p == 1 ? s1 : s2);
  const int h = p == 0 ? h0 : (p == 1 ? h1 : h2);
  void* redirect = pick3(e.out, p);
  const bool rope = (e.rope_mask >> p) & 1;
  if (!redirect && !rope) return;
  int64_t row = tok;
  if (redirect) {
    row = e.out_rows[tok];
    if (row < 0 || row >= e.out_rows_limit) {
      if (threadIdx.x == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
      return;
    }
  }
  const T* src = y + tok * ys;
  T* dst = redirect ? reinterpret_cast<T*>(redirect) + row * pick3(e.out_stride, p) : y + tok * ys;
  const T* cosp = reinterpret_cast<const T*>(e.cos) + tok * e.cs_stride;
  const T* sinp = reinterpret_cast<const T*>(e.sin) + tok * e.cs_stride;
  const int half = head_dim / 2;
  if (rope) {
    // one thread per pair: both elements are read before either is written (in place when dst == src)
    for (int i = threadIdx.x; i < h / 2; i += blockDim.x) {
      const int head = i / half, d = i - head * half;
      const int o0 = head * head_dim + d, o1 = o0 + half;
      const float x0 = to_f32<T>(src[o0]), x1 = to_f32<T>(src[o1]);
      const float c = to_f32<T>(cosp[d]), s = to_f32<T>(sinp[d]);
      dst[o0] = from_f32<T>(fmaf(-x1, s, x0 * c));
      dst[o1] = from_f32<T>(fmaf(x0, s, x1 * c));
    }
  } else {
    for (int i = threadIdx.x; i < h; i += blockDim.x) dst[i] = src[i];
  }
}

}  // namespace slora
