// Tensor-core (tcgen05) LoRA shrink / expand kernels for long same-adapter segments (prefill).
//
// A prefill sequence gives hundreds of consecutive tokens that share one adapter: its shrink is the small GEMM
// delta[n x r] = X[n x h_in] * A^T and its expand y[n x h_out] += scale * delta[n x r] * B^T.  At rank 64 these run
// at ~45 flop per byte, beyond what the FP32 pipes sustain at HBM speed, so tiles of 128 tokens go to the 5th
// generation tensor cores: operands are staged in shared memory in the un-swizzled K-major core-matrix layout with
// 16-byte cp.async copies (token rows and pool rows are gathered through the same index tables as everywhere else,
// so no tensor map is needed), one thread issues tcgen05.mma with the accumulator in tensor memory, completion is
// tracked with tcgen05.commit on an mbarrier, and the epilogue reads the accumulator back with tcgen05.ld.
//
// Operand layout in shared memory (both operands, element size 2): the tile [rows x 8*chunks] is cut into 16-byte
// chunks (8 elements of K); chunk (row, c) lives at  c * rows * 16 + row * 16.  Eight consecutive rows of one chunk
// form a contiguous 128-byte core matrix, so the descriptor's stride between 8-row groups (SBO) is 128 bytes and
// the stride between the two K-chunks of one K=16 instruction (LBO) is rows * 16 bytes.
//
// Every wait is bounded; a CTA that gives up records SLORA_STATUS_TIMEOUT, drains its copies and frees its tensor
// memory before it returns.
#pragma once

#include "lora_pipelined.cuh"

namespace slora {

constexpr int kMmaTokens = 128;    // tokens per tile = M of one tcgen05.mma
constexpr int kMmaThreads = 128;   // four warps: warp w reads accumulator lanes [32w, 32w + 32)
constexpr int kMmaKBlock = 64;     // K elements staged per pipeline stage of the shrink
constexpr int kMmaKChunks = kMmaKBlock / 8;
constexpr int kMmaStages = 4;
constexpr int kMmaMinTokens = 32;  // segments at least this long are served here
constexpr int kMmaMaxRows = 256;   // adapter rows one shrink CTA multiplies by (N of the instruction)
constexpr int kMmaShrinkCols = 256;
constexpr int kMmaSlack = 8 * 1024;  // unused tail of the dynamic shared memory
constexpr int kMmaOutChunk = 128;    // outputs per accumulator tile of the expand
constexpr int kMmaOutPerCta = 512;   // outputs one expand CTA walks through
constexpr int kMmaExpandCols = 128;
constexpr int kMmaMaxRank = 128;
constexpr int kMmaXTileBytes = kMmaTokens * kMmaKBlock * 2;         // 16 KB
constexpr int kMmaOperandBytes = kMmaTokens * kMmaMaxRank * 2;      // 32 KB: [128 x 128] expand operand

// ---- PTX wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Tensor-memory allocation: issued by one whole warp; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The barrier receives one arrival when every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, one K=16 step of 16-bit inputs with FP32 accumulation.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 16 consecutive FP32 accumulator columns of this thread's lane (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: start address, LBO (K-chunk stride) and SBO (8-row group
// stride) in 16-byte units, descriptor version 1.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// Instruction descriptor: FP32 accumulator, A and B both of type T and K-major, M = 128, N = n.
template <typename T>
struct UmmaFormat;
template <>
struct UmmaFormat<__half> {
  static constexpr uint32_t value = 0;
};
template <>
struct UmmaFormat<__nv_bfloat16> {
  static constexpr uint32_t value = 1;
};
template <typename T>
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  const uint32_t fmt = UmmaFormat<T>::value;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kMmaTokens >> 4) << 24);
}

// ---- tiles ----------------------------------------------------------------------------------------------------
struct MmaTile {
  int adapter;
  int first;  // first token of the tile
  int n;      // tokens, 1..kMmaTokens
  int r;      // slot rows of the adapter
  int64_t loc_base;
};

// May the tensor-core kernels take a segment of `len` tokens whose adapter has `r` slot rows?  The CUDA-core kernels
// skip exactly the segments for which this holds (TileSrc::seg_split > 0), so the two launches partition the work.
__device__ __forceinline__ bool mma_serves(const TileSrc& s, const Tables& tb, int64_t len, int64_t r) {
  return s.seg_split > 0 && len >= s.seg_split && r >= 8 && r <= kMmaMaxRank && r % 8 == 0 && tb.pool_stride % r == 0;
}

__device__ __forceinline__ bool lookup_mma_tile(const TileSrc& s, const Tables& tb, int tile_idx, MmaTile& t,
                                                int32_t* status) {
  const int seg = tile_idx / s.mma_tiles_per_seg;
  const int sub = tile_idx - seg * s.mma_tiles_per_seg;
  if (seg >= s.n_seg) return false;
  const int64_t len = s.seg_len[seg];
  const int64_t off = static_cast<int64_t>(sub) * kMmaTokens;
  if (off >= len) return false;
  const int64_t first = static_cast<int64_t>(s.seg_start[seg]) + off;
  if (first < 0 || first >= s.T) return false;
  int64_t n = len - off;
  if (n > kMmaTokens) n = kMmaTokens;
  if (first + n > s.T) n = s.T - first;
  const int64_t adapter = s.ids[seg];
  // range errors are reported by the CUDA-core launch that accompanies this one
  if (adapter < 0 || adapter >= tb.n_adapters) return false;
  const int64_t r4 = tb.ranks4[adapter];
  const int64_t st = tb.start[adapter];
  if (r4 < 0 || st < 0 || st + r4 > tb.loc_len || r4 > (int64_t(1) << 20)) return false;
  if (!mma_serves(s, tb, len, r4 >> 2)) return false;
  (void)status;
  t.adapter = static_cast<int>(adapter);
  t.first = static_cast<int>(first);
  t.n = static_cast<int>(n);
  t.r = static_cast<int>(r4 >> 2);
  t.loc_base = st;
  return true;
}

// ------------------------------------------------------------------------------------------------------------
// shrink: delta[p][tok, j] = sum_k x[tok, k] * A_p[j, k] for the projections p of this CTA's group
// grid: (segment tile, projection group).  dynamic shared memory: kMmaStages stages of
//   [x tile 128 x 64][adapter rows npad_max x 64], then kMmaSlack unused bytes
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kMmaThreads, 1) lora_shrink_mma_kernel(const ShrinkArgs a) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ __align__(8) uint64_t mma_done[kMmaStages];
  __shared__ uint32_t s_tmem;

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pg = blockIdx.x % a.max_rb;
  const int tile_idx = blockIdx.x / a.max_rb;
  MmaTile t;
  if (!lookup_mma_tile(a.src, a.tb, tile_idx, t, nullptr)) return;
  const int r = t.r;
  const int gp = a.rows_per_cta;  // projections per CTA; their qkvo indices are consecutive
  const int p0 = pg * gp;
  const int rows = gp * r;
  const int npad = (rows + 15) & ~15;
  if (rows > kMmaMaxRows || kMmaXTileBytes + npad * (kMmaKBlock * 2) > a.mma_stage_bytes) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_RANK);  // wider than the caller's delta_width promised
    return;
  }
  const int64_t S = a.tb.pool_stride;
  const int64_t base = t.loc_base + static_cast<int64_t>(r) * pick3(a.qkvo, p0);

  // every adapter row this CTA reads is checked before anything is copied
  bool rows_ok = true;
  for (int j = tid; j < rows; j += kMmaThreads) {
    const int64_t e = a.tb.loc[base + j];
    if (e < 0 || e >= a.tb.pool_rows) rows_ok = false;
  }
  if (!__syncthreads_and(rows_ok)) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_TABLE);
    return;
  }

  // this thread's share of every stage: chunk c of eight token rows and of up to sixteen adapter rows
  const int c = (tid >> 3) & (kMmaKChunks - 1);
  const int row0 = ((tid >> 6) << 3) | (tid & 7);
  const T* xsrc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = row0 + i * 16;
    const int tok = t.first + min(row, t.n - 1);
    xsrc[i] = reinterpret_cast<const T*>(a.x) + static_cast<int64_t>(tok) * a.x_stride + c * 8;
  }
  const int na = npad >> 4;  // adapter-row copies per thread and stage
  const T* asrc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = min(row0 + i * 16, rows - 1);
    const int64_t e = (i < na) ? a.tb.loc[base + row] : 0;
    asrc[i] = reinterpret_cast<const T*>(a.w) + e * S + c * 8;
  }
  const uint32_t smem0 = smem_u32(dyn_smem);
  const uint32_t stage_bytes = static_cast<uint32_t>(a.mma_stage_bytes);
  const uint32_t x_dst = c * (kMmaTokens * 16) + row0 * 16;
  const uint32_t a_dst = kMmaXTileBytes + c * (npad * 16) + row0 * 16;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kMmaStages; ++s) mbar_init(&mma_done[s], 1);
    fence_barrier_init();
  }
  // accumulator columns: a power of two covering the widest tile of this launch
  const uint32_t cols = (a.mma_stage_bytes - kMmaXTileBytes) / (kMmaKBlock * 2) > 128 ? kMmaShrinkCols : 128;
  if (warp == 0) {
    tmem_alloc(&s_tmem, cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  const uint32_t idesc = umma_idesc<T>(npad);
  const int nkb = a.h_in / kMmaKBlock;

  pdl_wait();  // activations come from the kernel before this one
  bool ok = true;
  for (int kb = 0; kb < nkb + kMmaStages - 1; ++kb) {
    if (kb < nkb) {
      const int s = kb % kMmaStages;
      // the MMAs that read this stage's previous contents must have completed
      if (kb >= kMmaStages) ok = ok && mbar_wait_timed(&mma_done[s], ((kb / kMmaStages) - 1) & 1);
      if (ok) {
        const uint32_t sb = smem0 + s * stage_bytes;
        const int k0 = kb * kMmaKBlock;
#pragma unroll
        for (int i = 0; i < 8; ++i) cp_async16(sb + x_dst + i * 256, xsrc[i] + k0);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (i < na) cp_async16(sb + a_dst + i * 256, asrc[i] + k0);
        }
      }
    }
    cp_async_commit();
    const int kc = kb - (kMmaStages - 1);
    if (kc >= 0) {
      cp_async_wait<kMmaStages - 1>();
      fence_proxy_async();
      if (!__syncthreads_and(ok)) {
        ok = false;
        break;
      }
      if (tid == 0) {
        tc_fence_after();
        const uint32_t sb = smem0 + (kc % kMmaStages) * stage_bytes;
#pragma unroll
        for (int ks = 0; ks < kMmaKBlock / 16; ++ks) {
          const uint64_t da = umma_smem_desc(sb + ks * 2 * (kMmaTokens * 16), kMmaTokens * 16, 128);
          const uint64_t db = umma_smem_desc(sb + kMmaXTileBytes + ks * 2 * (npad * 16), npad * 16, 128);
          umma_f16(tmem, da, db, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&mma_done[kc % kMmaStages]);
      }
    }
  }
  cp_async_wait<0>();
  if (ok) ok = mbar_wait_timed(&mma_done[(nkb - 1) % kMmaStages], ((nkb - 1) / kMmaStages) & 1);
  ok = __syncthreads_and(ok);
  tc_fence_after();

  if (ok) {
    // epilogue: thread (warp, lane) owns accumulator lane 32 * warp + lane = one token of the tile
    const int row = warp * 32 + lane;
    const bool live = row < t.n;
    const int64_t tok = t.first + (live ? row : 0);
    bool vec = (r % 8 == 0) && (a.delta_stride % 8 == 0);
    for (int q = 0; q < gp; ++q) vec = vec && ((reinterpret_cast<uintptr_t>(pick3(a.delta, p0 + q)) & 15) == 0);
    int p = 0, jj = 0;  // column j = p * r + jj
    for (int c0 = 0; c0 < npad; c0 += 16) {
      uint32_t v[16];
      tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (c0 + h * 8 < rows) {
          T* drow = reinterpret_cast<T*>(pick3(a.delta, p0 + p)) + tok * a.delta_stride;
          if (vec) {
            if (live && jj + 8 <= a.delta_width) {
              union {
                uint4 q;
                T e[8];
              } pk;
#pragma unroll
              for (int e = 0; e < 8; ++e) pk.e[e] = from_f32<T>(__uint_as_float(v[h * 8 + e]));
              *reinterpret_cast<uint4*>(drow + jj) = pk.q;
            } else if (live) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                if (jj + e < a.delta_width) drow[jj + e] = from_f32<T>(__uint_as_float(v[h * 8 + e]));
              }
            }
            jj += 8;
            if (jj >= r) {
              jj = 0;
              ++p;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (c0 + h * 8 + e < rows) {
                if (live && jj < a.delta_width)
                  drow[jj] = from_f32<T>(__uint_as_float(v[h * 8 + e]));
                if (++jj >= r) {
                  jj = 0;
                  ++p;
                }
              }
            }
          }
        }
      }
    }
  } else if (tid == 0) {
    set_status(a.status, SLORA_STATUS_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, cols);
}

// ------------------------------------------------------------------------------------------------------------
// expand: y[p][tok, o] += scale * sum_k delta[p][tok, k] * B_p[o, k],  B_p[o, k] = flat slot element o * r + k
// grid: (segment tile, projection, range of kMmaOutPerCta outputs).  dynamic shared memory:
//   [delta tile 128 x kpad][B chunk stage 0: 128 x kpad][B chunk stage 1], 32 KB each, then kMmaSlack unused bytes
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kMmaThreads) lora_expand_mma_kernel(const ExpandArgs a) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ __align__(8) uint64_t acc_done;
  __shared__ uint32_t s_tmem;

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per_tile = a.chunk_begin[a.nproj];
  const int tile_idx = blockIdx.x / per_tile;
  int cidx = blockIdx.x - tile_idx * per_tile;
  int p = 0;
  while (p + 1 < a.nproj && cidx >= a.chunk_begin[p + 1]) ++p;
  cidx -= a.chunk_begin[p];
  MmaTile t;
  if (!lookup_mma_tile(a.src, a.tb, tile_idx, t, nullptr)) return;
  const int R = t.r;  // rank_mult == 1 on this path
  const int h_out = pick3(a.h_out, p);
  const int o_begin = cidx * kMmaOutPerCta;
  if (o_begin >= h_out) return;
  const int o_end = min(h_out, o_begin + kMmaOutPerCta);
  const int nch = (o_end - o_begin + kMmaOutChunk - 1) / kMmaOutChunk;
  const int64_t S = a.tb.pool_stride;
  const int64_t base = t.loc_base + static_cast<int64_t>(R) * pick3(a.qkvo, p);

  // the pool rows behind outputs [o_begin, o_end) are checked before anything is copied
  const int pr_first = static_cast<int>(static_cast<int64_t>(o_begin) * R / S);
  const int pr_last = static_cast<int>((static_cast<int64_t>(o_end) * R - 1) / S);
  bool rows_ok = true;
  for (int pr = pr_first + tid; pr <= pr_last; pr += kMmaThreads) {
    if (pr >= R) {
      rows_ok = false;
    } else {
      const int64_t e = a.tb.loc[base + pr];
      if (e < 0 || e >= a.tb.pool_rows) rows_ok = false;
    }
  }
  if (!__syncthreads_and(rows_ok)) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_TABLE);
    return;
  }

  const int cpr = R >> 3;             // 16-byte chunks per operand row
  const int kpad = (R + 15) & ~15;    // K of the contraction, zero-padded to the instruction's K = 16
  const uint32_t smem0 = smem_u32(dyn_smem);
  const uint32_t d_smem = smem0;
  const uint32_t b_smem = smem0 + kMmaOperandBytes;
  constexpr uint32_t kLbo = kMmaTokens * 16;  // both operands hold 128 rows

  // This thread's cpr copies of every operand tile: item id = it * 128 + tid -> (row, chunk).
  uint32_t item_dst[16];  // byte offset inside an operand tile
  uint32_t item_rel[16];  // row * R + chunk * 8
#pragma unroll
  for (int it = 0; it < 16; ++it) {
    const int id = it * kMmaThreads + tid;
    const int g = id / (8 * cpr);
    const int rem = id - g * (8 * cpr);
    const int ch = rem >> 3;
    const int row = g * 8 + (rem & 7);
    item_dst[it] = ch * kLbo + row * 16;
    item_rel[it] = (static_cast<uint32_t>(row) << 16) | static_cast<uint32_t>(ch);
  }
  if (kpad != R) {
    // the chunk that pads K to a multiple of 16 is zero in all three operand tiles and never overwritten
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int row = tid; row < 3 * kMmaTokens; row += kMmaThreads) {
      const int which = row / kMmaTokens;
      const int rr = row - which * kMmaTokens;
      *reinterpret_cast<uint4*>(dyn_smem + which * kMmaOperandBytes + cpr * kLbo + rr * 16) = z;
    }
  }

  auto load_b_chunk = [&](int ch_idx) {
    const int o0 = o_begin + ch_idx * kMmaOutChunk;
    const uint32_t dst = b_smem + (ch_idx & 1) * kMmaOperandBytes;
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      if (it < cpr) {
        const int row = static_cast<int>(item_rel[it] >> 16);
        const int chk = static_cast<int>(item_rel[it] & 0xffff);
        const int o = min(o0 + row, h_out - 1);
        const int64_t f = static_cast<int64_t>(o) * R + chk * 8;
        const int64_t pr = f / S;
        const int64_t col = f - pr * S;
        const int64_t e = a.tb.loc[base + pr];
        cp_async16(dst + item_dst[it], reinterpret_cast<const T*>(a.w) + e * S + col);
      }
    }
  };

  if (tid == 0) {
    mbar_init(&acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&s_tmem, kMmaExpandCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  load_b_chunk(0);  // the pool does not depend on the kernel before this one
  cp_async_commit();
  pdl_wait();
  {
    const T* dsrc = reinterpret_cast<const T*>(pick3(a.delta, p));
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      if (it < cpr) {
        const int row = static_cast<int>(item_rel[it] >> 16);
        const int chk = static_cast<int>(item_rel[it] & 0xffff);
        const int64_t tok = t.first + min(row, t.n - 1);
        cp_async16(d_smem + item_dst[it], dsrc + tok * a.delta_stride + chk * 8);
      }
    }
  }
  cp_async_commit();

  const float scale = to_f32<T>(reinterpret_cast<const T*>(a.scales)[t.adapter]);
  const int row = warp * 32 + lane;
  const bool live = row < t.n;
  T* yrow = reinterpret_cast<T*>(pick3(a.y, p)) + (t.first + (live ? row : 0)) * pick3(a.y_stride, p);
  bool ok = true;
  for (int ch = 0; ch < nch; ++ch) {
    if (ch + 1 < nch) load_b_chunk(ch + 1);
    cp_async_commit();
    const int o0 = o_begin + ch * kMmaOutChunk;
    const int ncols = min(kMmaOutChunk, o_end - o0);  // a multiple of 8
    const int npad = (ncols + 15) & ~15;
    // this token's 128 outputs of y, fetched while the operands land and the MMA runs
    uint4 yv[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      yv[q] = make_uint4(0, 0, 0, 0);
      if (live && q * 8 < ncols) yv[q] = *reinterpret_cast<const uint4*>(yrow + o0 + q * 8);
    }
    cp_async_wait<1>();
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc<T>(npad);
      const uint32_t bs = b_smem + (ch & 1) * kMmaOperandBytes;
      for (int ks = 0; ks < kpad / 16; ++ks) {
        const uint64_t da = umma_smem_desc(d_smem + ks * 2 * kLbo, kLbo, 128);
        const uint64_t db = umma_smem_desc(bs + ks * 2 * kLbo, kLbo, 128);
        umma_f16(tmem, da, db, idesc, ks > 0 ? 1u : 0u);
      }
      umma_commit(&acc_done);
    }
    ok = mbar_wait_timed(&acc_done, ch & 1);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
#pragma unroll
    for (int g = 0; g < kMmaOutChunk / 16; ++g) {
      if (g * 16 < npad) {  // uniform over the CTA
        uint32_t v[16];
        tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + g * 16, v);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int q = g * 2 + h;
          if (live && q * 8 < ncols) {
            union {
              uint4 q4;
              T e[8];
            } pk;
            pk.q4 = yv[q];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              pk.e[e] = from_f32<T>(fmaf(scale, __uint_as_float(v[h * 8 + e]), to_f32<T>(pk.e[e])));
            *reinterpret_cast<uint4*>(yrow + o0 + q * 8) = pk.q4;
          }
        }
      }
    }
    // all warps have read the accumulator before the next chunk's MMA overwrites it
    tc_fence_before();
    __syncthreads();
  }
  cp_async_wait<0>();
  if (!ok && tid == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kMmaExpandCols);
}

}  // namespace slora
