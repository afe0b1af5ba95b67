// Tensor-core (tcgen05) LoRA shrink / expand kernels for long same-adapter segments (prefill).
//
// A prefill sequence gives hundreds of consecutive tokens that share one adapter: its shrink is the small GEMM
// delta[n x r] = X[n x h_in] * A^T and its expand y[n x h_out] += scale * delta[n x r] * B^T.  At rank 64 these run
// at ~45 flop per byte, beyond what the FP32 pipes sustain at HBM speed, so tiles of 128 tokens go to the 5th
// generation tensor cores.  Both kernels are warp-specialised:
//
//   shrink   one lane issues TMA tile loads of the activations (tensor map over x, 128-byte swizzle), eight loader
//            warps gather the adapter rows through the index tables with 16-byte cp.async copies (one K-block in
//            flight per warp, so the proxy fence each warp needs after its copies never stalls another warp's),
//            one lane issues tcgen05.mma with the accumulator in tensor memory and frees stages with
//            tcgen05.commit, four warps read the accumulator back with tcgen05.ld and store delta.
//   expand   two loader warps gather chunks of 128 outputs of B with cp.async, one lane issues the MMAs into a
//            double-buffered accumulator, four warps scale and round the result into a swizzled shared-memory tile
//            that one lane adds into y with a TMA reduce (an element-wise 16-bit add in L2, which is also how the
//            reference accumulates: it rounds the FP32 sum to the output type and then adds, bgmv_impl.cuh:185-199).
//
// Operand layouts in shared memory.  Gathered operands (adapter rows, B chunks, delta tile) use the un-swizzled
// K-major core-matrix layout: the tile [rows x 8*chunks] is cut into 16-byte chunks (8 elements of K); chunk
// (row, c) lives at c * rows * 16 + row * 16, so eight consecutive rows of one chunk form a contiguous 128-byte
// core matrix, the descriptor's stride between 8-row groups (SBO) is 128 bytes and the stride between the two
// K-chunks of one K=16 instruction (LBO) is rows * 16 bytes.  TMA-loaded activations use the 128-byte swizzled
// K-major layout (rows of 64 elements, SBO = 1024 bytes, K advanced by 32 bytes inside the swizzle span).
//
// Every wait is bounded; a CTA that gives up records SLORA_STATUS_TIMEOUT and frees its tensor memory before it
// returns.  No load uses cluster multicast.
#pragma once

#include <cuda.h>

#include "lora_pipelined.cuh"

namespace slora {

constexpr int kMmaTokens = 128;    // tokens per tile = M of one tcgen05.mma
constexpr int kMmaKBlock = 64;     // K elements per pipeline stage of the shrink (one 128-byte swizzle span)
constexpr int kMmaMinTokens = kBigSegmentTokens;  // segments at least this long are served here
constexpr int kMmaMaxRows = 256;   // adapter rows one shrink CTA multiplies by (N of the instruction)
constexpr int kMmaMaxRank = 128;
constexpr int kMmaMaxStages = 8;
constexpr int kMmaLoaderWarps = 8;  // shrink: one stage per loader warp
constexpr int kMmaShrinkThreads = (kMmaLoaderWarps + 2) * 32;  // + activation TMA warp + MMA warp
constexpr int kMmaXTileBytes = kMmaTokens * kMmaKBlock * 2;    // 16 KB
constexpr int kMmaSmemBudget = 200 * 1024;
constexpr int kMmaOutChunk = 128;   // outputs per accumulator tile of the expand
constexpr int kMmaOutPerCta = 512;  // outputs one expand CTA walks through
constexpr int kMmaExLoaderWarps = 2;
constexpr int kMmaExStages = 2;
constexpr int kMmaExpandThreads = (4 + kMmaExLoaderWarps + 1) * 32;
constexpr int kMmaOutRowPitch = kMmaOutChunk * 2 + 16;  // gathered tokens: one padded row per token (no bank conflicts)
constexpr int kMmaOutTileBytes = 35 * 1024;  // two swizzled 16 KB halves of 64 columns, or 128 rows of kMmaOutRowPitch
constexpr int kMmaExpandCols = 256;                              // two accumulators of 128 columns

// Tensor maps of the y buffers of one expand call.
struct TmapSet {
  CUtensorMap m[3];
};

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

// TMA tile load (2-D tensor map) into this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Bulk reduce of one contiguous run: global[i] += shared[i] for `bytes` bytes of T elements (both addresses 16-byte
// aligned, bytes a multiple of 16); completion is tracked by the issuing thread's bulk group.
template <typename T>
__device__ __forceinline__ void bulk_reduce_add(void* dst, uint32_t src, uint32_t bytes);
template <>
__device__ __forceinline__ void bulk_reduce_add<__half>(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;" ::"l"(dst), "r"(src),
               "r"(bytes)
               : "memory");
}
template <>
__device__ __forceinline__ void bulk_reduce_add<__nv_bfloat16>(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(dst), "r"(src),
               "r"(bytes)
               : "memory");
}
// TMA tile reduce: global[tile] += shared[tile], element-wise in the tensor map's type.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Thread-block cluster helpers (split-K shrink): this CTA's rank, a barrier over all threads of the cluster, the
// address of a peer CTA's copy of a shared-memory location, and a 16-byte load from it.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_peer_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ int ld_peer_i32(uint32_t addr) {
  int v;
  asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Barrier among `threads` threads of the CTA (hardware barrier 1; barrier 0 is __syncthreads), and the same with an
// AND-reduction of a predicate.
__device__ __forceinline__ void named_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }
__device__ __forceinline__ bool named_and(int threads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.and.pred p, 1, %2, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(pred)), "r"(threads)
      : "memory");
  return out != 0;
}
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t addr) {
  uint64_t d = static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// ---- tiles ----------------------------------------------------------------------------------------------------
struct MmaTile {
  int adapter;
  int first;  // first token of the tile (segments) or first slot in perm (plan)
  int n;      // tokens, 1..kMmaTokens
  int r;      // slot rows of the adapter
  int64_t loc_base;
  const int32_t* perm;  // plan only: token of slot i is perm[first + i]; null when the tile's tokens are consecutive
};

// Token index of row `i` of a tile (rows beyond the tile's tokens repeat its last token).
__device__ __forceinline__ int64_t mma_token(const MmaTile& t, int i) {
  const int j = t.first + min(i, t.n - 1);
  return t.perm ? t.perm[j] : j;
}

// May the tensor-core kernels take a segment of `len` tokens whose adapter has `r` slot rows?  The CUDA-core kernels
// skip exactly the segments for which this holds (TileSrc::seg_split > 0), so the two launches partition the work.
__device__ __forceinline__ bool mma_serves(const TileSrc& s, const Tables& tb, int64_t len, int64_t r) {
  return s.seg_split > 0 && len >= s.seg_split && r >= 8 && r <= kMmaMaxRank && r % 8 == 0 && tb.pool_stride % r == 0 &&
         r <= s.mma_max_rows;
}

__device__ __forceinline__ bool lookup_mma_tile(const TileSrc& s, const Tables& tb, int tile_idx, MmaTile& t,
                                                int32_t* status) {
  if (s.mode == MODE_PLAN) {
    // big-tile records were validated by the plan builder
    const int32_t* hdr = s.plan;
    if (s.seg_split <= 0 || tile_idx >= hdr[PH_NBIG]) return false;
    const int4* rec = reinterpret_cast<const int4*>(s.plan + hdr[PH_BIGOFF] + kTileWords * tile_idx);
    const int4 r0 = rec[0];
    const int4 r1 = rec[1];
    t.adapter = r0.x;
    t.first = r0.y;
    t.n = r0.z;
    t.r = r0.w;
    t.loc_base = r1.x;
    t.perm = s.plan + PH_WORDS + kTileWords * hdr[PH_MAXTILES];
    return t.n > 0 && t.r > 0 && tb.pool_stride % t.r == 0 && t.r <= s.mma_max_rows;
  }
  t.perm = nullptr;
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
// grid: (segment tile, projection group).  dynamic shared memory (1024-byte aligned): `mma_stages` stages of
//   [x tile 128 x 64, swizzled][adapter rows npad_max x 64, core-matrix layout]
// ------------------------------------------------------------------------------------------------------------
struct ShrinkMmaCtl {
  uint64_t full[kMmaMaxStages];   // arrivals: the stage's loader warp and, for consecutive tokens, the activation
                                  // TMA (with its bytes); gathered tokens are copied by the loader warp itself
  uint64_t empty[kMmaMaxStages];  // 1 arrival: tcgen05.commit after the stage's MMAs
  uint64_t acc_done;
  uint32_t tmem;
  int bad;
  int64_t row_off[kMmaMaxRows];  // element offset of each adapter row in the pool
  int64_t tok_off[kMmaTokens];   // gathered tokens: element offset of each token row in x
};

template <typename T>
__global__ void __launch_bounds__(kMmaShrinkThreads, 1)
    lora_shrink_mma_kernel(const ShrinkArgs a, const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ __align__(1024) unsigned char mma_smem[];
  __shared__ ShrinkMmaCtl ctl;

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // split-K: the `ks` CTAs of a cluster share one (tile, projection group) and take consecutive K ranges; every
  // early return below depends on the tile only, so the CTAs of a cluster take it together
  const int ks = a.mma_ksplit;
  const int kq = ks > 1 ? static_cast<int>(cluster_rank()) : 0;
  const int unit = blockIdx.x / ks;
  const int pg = unit % a.max_rb;
  const int tile_idx = unit / a.max_rb;
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
  for (int j = tid; j < npad; j += kMmaShrinkThreads) {
    const int64_t e = a.tb.loc[base + min(j, rows - 1)];
    if (e < 0 || e >= a.tb.pool_rows) rows_ok = false;
    ctl.row_off[j] = e * S;
  }
  const bool gather = t.perm != nullptr;
  if (gather) {
    for (int i = tid; i < kMmaTokens; i += kMmaShrinkThreads) ctl.tok_off[i] = mma_token(t, i) * a.x_stride;
  }
  if (!__syncthreads_and(rows_ok)) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_TABLE);
    return;
  }

  const int nst = a.mma_stages;
  const uint32_t smem0 = (smem_u32(mma_smem) + 1023u) & ~1023u;
  const uint32_t stage_bytes = static_cast<uint32_t>(a.mma_stage_bytes);
  const int nkb = a.h_in / kMmaKBlock / ks;  // K-blocks of this CTA
  const int kb_base = kq * nkb;
  if (tid == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(&ctl.full[s], gather ? 1 : 2);
      mbar_init(&ctl.empty[s], 1);
    }
    mbar_init(&ctl.acc_done, 1);
    ctl.bad = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  // accumulator columns: a power of two covering the widest tile of this launch
  const uint32_t cols = (a.mma_stage_bytes - kMmaXTileBytes) / (kMmaKBlock * 2) > 128 ? 256 : 128;
  if (warp == 0) {
    tmem_alloc(&ctl.tmem, cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem;

  if (warp < kMmaLoaderWarps) {
    // ---- loader warp: gathers the adapter rows of K-blocks warp, warp + nst, ... into stage `warp` ----
    if (warp < nst) {
      const int row_lo = lane & 7, c_lo = lane >> 3;
      const T* w = reinterpret_cast<const T*>(a.w);
      const T* x = reinterpret_cast<const T*>(a.x);
      const uint32_t dst0 = smem0 + warp * stage_bytes + kMmaXTileBytes + row_lo * 16;
      if (gather) pdl_wait();  // this warp reads the activations itself
      for (int kb = warp, use = 0; kb < nkb; kb += nst, ++use) {
        if (use > 0 && !mbar_wait_timed(&ctl.empty[warp], (use - 1) & 1)) {
          ctl.bad = 1;
          break;
        }
        const int k0 = (kb_base + kb) * kMmaKBlock;
        if (gather) {
          // token rows into the 128-byte swizzled layout the TMA would have produced: chunk c of row i at
          // i * 128 + ((c ^ (i & 7)) << 4)
          const uint32_t xdst = smem0 + warp * stage_bytes;
          for (int rg = 0; rg < kMmaTokens; rg += 8) {
            const int row = rg + row_lo;
            const T* src = x + ctl.tok_off[row] + k0;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
              const int c = ch * 4 + c_lo;
              cp_async16(xdst + row * 128 + ((c ^ row_lo) << 4), src + c * 8);
            }
          }
        }
        for (int rg = 0; rg < npad; rg += 8) {
          const T* src = w + ctl.row_off[rg + row_lo] + k0;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int c = ch * 4 + c_lo;
            cp_async16(dst0 + c * (npad * 16) + rg * 16, src + c * 8);
          }
        }
        cp_async_wait_all();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.full[warp]);
      }
    }
  } else if (warp == kMmaLoaderWarps) {
    // ---- activation tiles by TMA (consecutive tokens only) ----
    if (lane == 0 && !gather) {
      pdl_wait();  // activations come from the kernel before this one
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % nst, use = kb / nst;
        if (use > 0 && !mbar_wait_timed(&ctl.empty[s], (use - 1) & 1)) {
          ctl.bad = 1;
          break;
        }
        mbar_expect_tx(&ctl.full[s], kMmaXTileBytes);
        tma_load_2d(smem0 + s * stage_bytes, &x_map, (kb_base + kb) * kMmaKBlock, t.first, &ctl.full[s]);
      }
    }
  } else {
    // ---- MMA issue ----
    if (lane == 0) {
      const uint32_t idesc = umma_idesc<T>(npad);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % nst, use = kb / nst;
        if (!mbar_wait_timed(&ctl.full[s], use & 1)) {
          ctl.bad = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sb = smem0 + s * stage_bytes;
#pragma unroll
        for (int ks = 0; ks < kMmaKBlock / 16; ++ks) {
          const uint64_t da = umma_smem_desc_sw128(sb + ks * 32);
          const uint64_t db = umma_smem_desc(sb + kMmaXTileBytes + ks * 2 * (npad * 16), npad * 16, 128);
          umma_f16(tmem, da, db, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&ctl.empty[s]);
      }
      if (ok) umma_commit(&ctl.acc_done);
    }
  }

  // ---- epilogue: thread (warp, lane) of warps 0..3 owns accumulator lane 32 * warp + lane = one token ----
  bool ok = true;
  if (warp < 4) ok = mbar_wait_timed(&ctl.acc_done, 0);
  ok = __syncthreads_and(ok) && ctl.bad == 0;
  tc_fence_after();
  bool vec = (a.delta_stride % 8 == 0);
  for (int q = 0; q < gp; ++q) vec = vec && ((reinterpret_cast<uintptr_t>(pick3(a.delta, p0 + q)) & 15) == 0);
  // eight consecutive columns [j0, j0 + 8) of row `tok` (j0 a multiple of 8, so they lie in one projection)
  auto store8 = [&](int64_t tok, int j0, const float (&f)[8]) {
    const int p = j0 / r, jj = j0 - p * r;
    T* drow = reinterpret_cast<T*>(pick3(a.delta, p0 + p)) + tok * a.delta_stride;
    if (vec && jj + 8 <= a.delta_width) {
      union {
        uint4 q;
        T e[8];
      } pk;
#pragma unroll
      for (int e = 0; e < 8; ++e) pk.e[e] = from_f32<T>(f[e]);
      *reinterpret_cast<uint4*>(drow + jj) = pk.q;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (jj + e < a.delta_width) drow[jj + e] = from_f32<T>(f[e]);
      }
    }
  };
  if (ks == 1) {
    if (ok && warp < 4) {
      const int row = warp * 32 + lane;
      const bool live = row < t.n;
      const int64_t tok = mma_token(t, live ? row : 0);
      for (int c0 = 0; c0 < npad; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (live && c0 + h * 8 < rows) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[h * 8 + e]);
            store8(tok, c0 + h * 8, f);
          }
        }
      }
    }
  } else {
    // partial sums to shared memory (the pipeline stages are idle now): [128 rows][npad + 4] floats
    const uint32_t pitch = static_cast<uint32_t>(npad + 4) * 4;
    if (ok && warp < 4) {
      const int row = warp * 32 + lane;
      for (int c0 = 0; c0 < npad; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 4; ++h)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem0 + row * pitch + (c0 + h * 4) * 4),
                       "r"(v[h * 4]), "r"(v[h * 4 + 1]), "r"(v[h * 4 + 2]), "r"(v[h * 4 + 3])
                       : "memory");
      }
    }
    if (tid == 0 && !ok) ctl.bad = 1;
    cluster_sync_all();
    // CTA kq adds the ks partial tiles for its share of the rows, in rank order, and stores them
    bool all_ok = true;
    for (int q = 0; q < ks; ++q) all_ok = all_ok && ld_peer_i32(peer_smem(smem_u32(&ctl.bad), q)) == 0;
    if (all_ok && tid < 128) {
      const int rows_per = kMmaTokens / ks;
      const int groups = npad >> 3;
      for (int u = tid; u < rows_per * groups; u += 128) {
        const int row = kq * rows_per + u / groups;
        const int j0 = (u % groups) * 8;
        if (row < t.n && j0 < rows) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = 0.f;
          const uint32_t local = smem0 + row * pitch + j0 * 4;
          for (int q = 0; q < ks; ++q) {
            const uint32_t pa = peer_smem(local, q);
            const float4 lo4 = ld_peer_f4(pa), hi4 = ld_peer_f4(pa + 16);
            f[0] += lo4.x, f[1] += lo4.y, f[2] += lo4.z, f[3] += lo4.w;
            f[4] += hi4.x, f[5] += hi4.y, f[6] += hi4.z, f[7] += hi4.w;
          }
          store8(mma_token(t, row), j0, f);
        }
      }
    }
    ok = all_ok;
    // no CTA of the cluster may leave while a peer still reads its shared memory
    cluster_sync_all();
  }
  if (!ok && tid == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, cols);
}

// ------------------------------------------------------------------------------------------------------------
// expand: y[p][tok, o] += scale * sum_k delta[p][tok, k] * B_p[o, k],  B_p[o, k] = flat slot element o * r + k
// grid: (segment tile, projection, range of kMmaOutPerCta outputs).  dynamic shared memory (1024-byte aligned):
//   [out tile] 32 KB (two 128-byte-swizzled halves of 64 columns),
//   [delta tile 128 x kpad_max][B chunk stage 0][B chunk stage 1] of `mma_stage_bytes` each (core-matrix layout)
// ------------------------------------------------------------------------------------------------------------
struct ExpandMmaCtl {
  uint64_t d_full;                    // arrivals: the loader warps (delta tile landed)
  uint64_t b_full[kMmaExStages];      // 1 arrival: the chunk's loader warp
  uint64_t b_empty[kMmaExStages];     // 1 arrival: tcgen05.commit
  uint64_t acc_full[2];               // 1 arrival: tcgen05.commit
  uint64_t acc_empty[2];              // 4 arrivals: the epilogue warps
  uint32_t tmem;
  int bad;
};

template <typename T>
__global__ void __launch_bounds__(kMmaExpandThreads)
    lora_expand_mma_kernel(const ExpandArgs a, const __grid_constant__ TmapSet y_maps) {
  extern __shared__ __align__(1024) unsigned char mma_smem[];
  __shared__ ExpandMmaCtl ctl;
  __shared__ int64_t s_row_off[kMmaOutPerCta * kMmaMaxRank / 8 / 8 + 2];  // pool rows behind this CTA's outputs

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
  const uint32_t S = static_cast<uint32_t>(a.tb.pool_stride);
  const int64_t base = t.loc_base + static_cast<int64_t>(R) * pick3(a.qkvo, p);
  const int kpad = (R + 15) & ~15;  // K of the contraction, zero-padded to the instruction's K = 16
  const uint32_t tile_bytes = static_cast<uint32_t>(a.mma_stage_bytes);
  if (static_cast<uint32_t>(kMmaTokens * kpad * 2) > tile_bytes) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_RANK);  // wider than the caller's delta_width promised
    return;
  }

  // the pool rows behind outputs [o_begin, o_end) are checked before anything is copied
  const uint32_t pr_first = static_cast<uint32_t>(o_begin) * R / S;
  const uint32_t pr_last = (static_cast<uint32_t>(o_end) * R - 1) / S;
  bool rows_ok = pr_last - pr_first < sizeof(s_row_off) / sizeof(s_row_off[0]);
  for (uint32_t pr = pr_first + tid; pr <= pr_last && rows_ok; pr += kMmaExpandThreads) {
    if (pr >= static_cast<uint32_t>(R)) {
      rows_ok = false;
    } else {
      const int64_t e = a.tb.loc[base + pr];
      if (e < 0 || e >= a.tb.pool_rows) rows_ok = false;
      s_row_off[pr - pr_first] = e * static_cast<int64_t>(S);
    }
  }
  if (!__syncthreads_and(rows_ok)) {
    if (tid == 0) set_status(a.status, SLORA_STATUS_BAD_TABLE);
    return;
  }

  const int cpr = R >> 3;  // 16-byte chunks per operand row
  const uint32_t smem0 = (smem_u32(mma_smem) + 1023u) & ~1023u;
  const uint32_t out_smem = smem0;
  const uint32_t d_smem = smem0 + kMmaOutTileBytes;
  const uint32_t b_smem = d_smem + tile_bytes;
  constexpr uint32_t kLbo = kMmaTokens * 16;  // both operands hold 128 rows

  if (tid == 0) {
    mbar_init(&ctl.d_full, kMmaExLoaderWarps);
    for (int s = 0; s < kMmaExStages; ++s) {
      mbar_init(&ctl.b_full[s], 1);
      mbar_init(&ctl.b_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl.acc_full[s], 1);
      mbar_init(&ctl.acc_empty[s], 4);
    }
    ctl.bad = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) {
    tmem_alloc(&ctl.tmem, kMmaExpandCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem;

  if (warp < 4) {
    // ---- epilogue: scale, round, stage in shared memory, add into y with a TMA reduce (consecutive tokens: one
    // tile reduce per 64 columns; gathered tokens: one bulk reduce per token row, issued by the row's own thread) ----
    const float scale = to_f32<T>(reinterpret_cast<const T*>(a.scales)[t.adapter]);
    const int row = warp * 32 + lane;
    const bool live = row < t.n;
    const bool gather = t.perm != nullptr;
    const CUtensorMap* ymap = &y_maps.m[p];
    T* yrow = reinterpret_cast<T*>(pick3(a.y, p)) + mma_token(t, live ? row : 0) * pick3(a.y_stride, p);
    pdl_wait();  // y is also written by the kernel before this one
    for (int ch = 0; ch < nch; ++ch) {
      const int ab = ch & 1;
      const int o0 = o_begin + ch * kMmaOutChunk;
      const int ncols = min(kMmaOutChunk, o_end - o0);  // a multiple of 8
      const int npad = (ncols + 15) & ~15;
      // the previous chunk's reduce must have finished reading the out tile
      if (gather || tid == 0) bulk_wait_read<0>();
      const bool got = mbar_wait_timed(&ctl.acc_full[ab], (ch >> 1) & 1);
      // all four warps go on, or leave, together
      if (!named_and(128, got)) {
        ctl.bad = 1;
        break;
      }
      tc_fence_after();
      const uint32_t out_tile = out_smem;
#pragma unroll
      for (int g = 0; g < kMmaOutChunk / 16; ++g) {
        if (g * 16 < npad) {  // uniform over the warps
          uint32_t v[16];
          tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + ab * kMmaOutChunk + g * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            union {
              uint4 q4;
              T e[8];
            } pk;
#pragma unroll
            for (int e = 0; e < 8; ++e)
              pk.e[e] = from_f32<T>(live ? scale * __uint_as_float(v[h * 8 + e]) : 0.f);
            const int col = g * 16 + h * 8;  // column of the 128-wide tile; half = col / 64
            const uint32_t cc = static_cast<uint32_t>((col & 63) >> 3);
            const uint32_t dst =
                gather ? out_tile + row * kMmaOutRowPitch + col * 2
                       : out_tile + (col >> 6) * (kMmaTokens * 128) + row * 128 + ((cc ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk.q4.x), "r"(pk.q4.y),
                         "r"(pk.q4.z), "r"(pk.q4.w)
                         : "memory");
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.acc_empty[ab]);
      fence_proxy_async();
      if (gather) {
        // each thread adds the row it wrote itself: no barrier needed
        if (live) bulk_reduce_add<T>(yrow + o0, out_tile + row * kMmaOutRowPitch, static_cast<uint32_t>(ncols) * 2);
        bulk_commit();
      } else {
        named_sync(128);
        if (tid == 0) {
          for (int half = 0; half * 64 < ncols; ++half)
            tma_reduce_add_2d(ymap, o0 + half * 64, t.first, out_tile + half * (kMmaTokens * 128));
          bulk_commit();
        }
      }
    }
    if (gather || tid == 0) bulk_wait<0>();
  } else if (warp < 4 + kMmaExLoaderWarps) {
    // ---- loader warps: the delta tile once, then B chunks lw, lw + 2, ... ----
    const int lw = warp - 4;
    const T* wsrc = reinterpret_cast<const T*>(a.w);
    const int n_items = kMmaTokens * cpr;
    if (kpad != R) {
      // the chunk that pads K to a multiple of 16 is zero in all operand tiles and never overwritten
      for (int i = lw * 32 + lane; i < 3 * kMmaTokens; i += kMmaExLoaderWarps * 32) {
        const int which = i / kMmaTokens, rr = i - which * kMmaTokens;
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(d_smem + which * tile_bytes + cpr * kLbo + rr * 16),
                     "r"(0u)
                     : "memory");
      }
    }
    for (int ch = lw, first = 1; ch < nch || first; ch += kMmaExLoaderWarps, first = 0) {
      if (ch < nch) {
        const int s = ch % kMmaExStages, use = ch / kMmaExStages;
        if (use > 0 && !mbar_wait_timed(&ctl.b_empty[s], (use - 1) & 1)) {
          ctl.bad = 1;
          break;
        }
        const int o0 = o_begin + ch * kMmaOutChunk;
        const uint32_t dst = b_smem + s * tile_bytes;
        for (int q = lane; q < n_items; q += 32) {
          const int row = q / cpr, c = q - row * cpr;
          const uint32_t o = static_cast<uint32_t>(min(o0 + row, h_out - 1));
          const uint32_t f = o * R + c * 8;
          const uint32_t pr = f / S, col = f - pr * S;
          cp_async16(dst + c * kLbo + row * 16, wsrc + s_row_off[pr - pr_first] + col);
        }
      }
      if (first) {
        pdl_wait();  // delta comes from the kernel before this one
        const T* dsrc = reinterpret_cast<const T*>(pick3(a.delta, p));
        for (int q = lw * 32 + lane; q < n_items; q += kMmaExLoaderWarps * 32) {
          const int row = q / cpr, c = q - row * cpr;
          cp_async16(d_smem + c * kLbo + row * 16, dsrc + mma_token(t, row) * a.delta_stride + c * 8);
        }
      }
      cp_async_wait_all();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (first) mbar_arrive(&ctl.d_full);
        if (ch < nch) mbar_arrive(&ctl.b_full[ch % kMmaExStages]);
      }
    }
  } else {
    // ---- MMA issue ----
    if (lane == 0) {
      bool ok = mbar_wait_timed(&ctl.d_full, 0);
      for (int ch = 0; ch < nch && ok; ++ch) {
        const int s = ch % kMmaExStages, use = ch / kMmaExStages, ab = ch & 1;
        ok = mbar_wait_timed(&ctl.b_full[s], use & 1);
        if (ok && ch >= 2) ok = mbar_wait_timed(&ctl.acc_empty[ab], ((ch >> 1) - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const int ncols = min(kMmaOutChunk, o_end - (o_begin + ch * kMmaOutChunk));
        const uint32_t idesc = umma_idesc<T>((ncols + 15) & ~15);
        const uint32_t bs = b_smem + s * tile_bytes;
        for (int ks = 0; ks < kpad / 16; ++ks) {
          const uint64_t da = umma_smem_desc(d_smem + ks * 2 * kLbo, kLbo, 128);
          const uint64_t db = umma_smem_desc(bs + ks * 2 * kLbo, kLbo, 128);
          umma_f16(tmem + ab * kMmaOutChunk, da, db, idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(&ctl.b_empty[s]);
        umma_commit(&ctl.acc_full[ab]);
      }
      if (!ok) ctl.bad = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctl.bad != 0 && tid == 0) set_status(a.status, SLORA_STATUS_TIMEOUT);
  if (warp == 0) tmem_dealloc(tmem, kMmaExpandCols);
}

}  // namespace slora
