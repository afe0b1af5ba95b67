// Shared definitions of the LoRA shrink / expand kernels: argument blocks, the batch-plan layout, tile lookup
// and the PTX wrappers (mbarrier, bulk asynchronous copy, programmatic dependent launch).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "slora_b200.h"

namespace slora {

constexpr int kTileTokens = 8;  // tokens per tile (plan granularity)
constexpr int kMaxRows = 4;     // adapter rows per shrink work item
constexpr int kChunk = 8192;    // flat B elements per expand work item (16 KB)
constexpr uint32_t kSpinLimit = 1u << 18;

// ---- batch plan workspace (int32 words) --------------------------------------------------------------------
//   [header PH_WORDS][tile records 8 * max_tiles][perm T][pos T][cnt n_adapters][big-tile records 8 * max_big]
// tile record: {adapter, first slot in perm, tokens (0 = skip), slot_rows r, first loc entry, big, 0, 0}
//   big = 1 when the tile's adapter has kBigGroupTokens tokens or more in the batch and 8..128 slot rows (a multiple
//   of 8): such groups are also listed as big tiles of up to 128 tokens for the tensor-core kernels
// big-tile record: {adapter, first slot in perm, tokens, slot_rows r, first loc entry, 0, 0, 0}
constexpr int PH_MAGIC = 0, PH_NTILES = 1, PH_STATUS = 2, PH_MAXTILES = 3, PH_T = 4, PH_NADAPTERS = 5, PH_NBIG = 6,
              PH_BIGOFF = 7, PH_MAXBIG = 8, PH_UNIFORM = 9;  // PH_UNIFORM: the slot rows every non-empty tile has, 0 when they differ
// PH_NSMALL: 8-token tiles of groups that are not big (the CUDA-core kernels' share when big groups go to the tensor
// cores); PH_BIG_RMAX: widest rank among the big groups; PH_BIG_POW2: 1 when every big group's rank is a power of two
constexpr int PH_NSMALL = 10, PH_BIG_RMAX = 11, PH_BIG_POW2 = 12;
// Resolved tiles (optional; a plan built with the adapters' loc table and a rank cap): after the big-tile records,
// one entry of kXtHead + 4 * cap words per tile slot: {token ids of the tile [8]; the adapter's scale (its 16 bits as
// stored in the table), 0, 0, 0; pool rows of projection 0 [cap], of projection 1 [cap], 2, 3} - everything a launch
// would otherwise chase through perm, the scale table and the loc table, at an
// address that follows from the tile index alone, so a producer can fetch the record and what hangs off it in one
// round trip.  PH_XOFF = word offset of the entries (0: none), PH_XRCAP = cap; tile record word 6 = 1 when the
// tile's entry is filled (rank <= cap).  A pool row that does not fit 31 bits is stored as -1 (the range check
// that follows every lookup refuses it).
constexpr int PH_XOFF = 13, PH_XRCAP = 14;
constexpr int kXtHead = 12;
constexpr int kBigGroupTokens = 128;  // planned batches: same-adapter groups at least this long go to the tensor cores
constexpr int kBigSegmentTokens = 32;  // segment calls: segments at least this long do
constexpr int kBigTileTokens = 128;
constexpr int PH_WORDS = 16;
constexpr int kTileWords = 8;
constexpr int32_t kPlanMagic = 0x534c5034;  // "SLP4"

enum TileMode { MODE_TOKEN = 0, MODE_PLAN = 1, MODE_SEGMENT = 2 };

struct TileSrc {
  const int32_t* plan;
  const int64_t* ids;  // TOKEN: adapter per token; SEGMENT: adapter per segment
  const int32_t* seg_start;
  const int32_t* seg_len;
  int mode;
  int n_seg;
  int tiles_per_seg;
  int slots;  // tile slots the launch enumerates (upper bound of the number of tiles)
  int seg_split;          // > 0 when segments (SEGMENT) / groups (PLAN) at least this long go to the tensor-core kernels
  int mma_tiles_per_seg;  // SEGMENT: 128-token tiles enumerated per segment by the tensor-core kernels
  int big_slots;          // PLAN: big-tile slots the tensor-core launch enumerates
  int big_exact;          // PLAN: big_slots is the plan's own count (host side), not an upper bound
  int mma_max_rows;       // adapters with more slot rows than this (the call's delta width) stay on the CUDA cores
  int xoff, xrcap;        // PLAN: where the host expects resolved tiles and their rank cap (0: do not look for them)
  int64_t T;
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

// One tile as the kernels see it.
struct TileInfo {
  int adapter;
  int first;  // PLAN: first slot in perm; otherwise first token
  int n;      // tokens, 1..kTileTokens
  int r;      // slot rows (= LoRA rank of the adapter as stored in the tables)
  int64_t loc_base;
  const int32_t* perm;  // PLAN only
  // PLAN with resolved tiles (TileSrc::xoff > 0): xt = this tile's entry, fetched without waiting for the header or
  // the record (the address follows from the tile index); xok = header and record confirm that the entry is there
  const int32_t* xt;
  int xrcap;
  bool xok;
  int tok[kTileTokens];  // the entry's token ids (valid when xok)
};

// Tensor-parallel link of a pipelined shrink (writes its result into every rank's delta buffer and signals) or expand
// (waits for every rank's signal before it reads its delta buffer).  See tp_exchange_kernel for the buffers.
constexpr int kTpMaxParts = 8;
struct TpLink {
  void* full[kTpMaxParts];       // shrink: every rank's delta buffer [2][3][full_tokens][R]
  int32_t* flags[kTpMaxParts];   // shrink: every rank's flags [2][n_parts]; expand: only flags[my_part] is used
  int32_t* counter;              // CTA arrival counter of this launch (zero between launches)
  int32_t* seq_state;            // this rank's exchanges completed per half
  int64_t full_tokens;
  int my_part, n_parts, half;
  int enabled;
  int inband;  // 1: no flags; the expand recognises delta values that have not arrived yet (see tp_has_empty)
               // 2: the same, and the expand does not wait for the shrink's grid either: this GPU's own values are
               //    recognised like the peers'.  The shrink then lets its dependents launch only after its own
               //    grid-dependency wait, so what came before the shrink (the base projection that wrote y) is
               //    complete before a CTA of the expand exists, and every CTA of the shrink is running by then.
               // 3: early start over rotating thirds.  The buffers hold three parts instead of two halves; exchange
               //    number e (kept on the device: seq_state[0] is read by a shrink after its grid-dependency wait,
               //    seq_state[1] is left by that shrink for its expand, which writes e + 1 back for the next
               //    shrink) works in part e % 3, and its SHRINK refills - spread over all CTAs, on this GPU's own
               //    buffer - the part that exchange e - 1 used, whose expand on this GPU is complete by then.  No
               //    arrival counter and no refill at the end of an expand.  A peer writes into that part again in
               //    exchange e + 2, i.e. after it has received all of this GPU's values of exchange e + 1, whose
               //    shrink starts writing after this GPU's expand e, which follows shrink e in stream order: the
               //    refill is a whole kernel ahead of the next write.  `half` is not used.
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
  int rank_mult;     // A rows per slot row (1 in the reference layout; N when a rank holds [r, h_in / N] slices)
  int max_rb;        // row blocks enumerated per (tile, projection)
  int rows_per_cta;  // <= kMaxRows
  int tok_pass;      // simple kernel: tokens staged per pass
  int piece;         // simple kernel: elements per bulk copy
  int mma_stage_bytes;  // tensor-core kernel: bytes of one pipeline stage
  int mma_stages;       // tensor-core kernel: pipeline stages
  int mma_ksplit;       // tensor-core kernel: CTAs (one cluster) that split K of one tile
  TpLink tp;
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
  int max_rank;  // widest rank the delta buffers hold (delta_width * delta_parts): wider adapters are refused
  int piece;  // elements per bulk copy (power of two dividing pool_stride, <= kChunk)
  int mma_stage_bytes;  // tensor-core kernel: bytes of one operand tile [128 x kpad_max]
  TpLink tp;
  int32_t* status;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------------------
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One probe of a barrier phase.  mbarrier.try_wait lets the hardware park the warp for a short, system-dependent time
// when the phase has not flipped yet, so a waiting warp takes few issue slots from the warps that share its
// scheduler (with test_wait, which never parks, three quarters of a decode launch's instructions were spin-loop
// instructions; measured 1 to 3 % less time per layer with try_wait).  SLORA_WAIT_SPIN builds the test_wait form.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
#ifdef SLORA_WAIT_SPIN
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
#endif
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: true when the phase completed within the limit (a number of probes and, because a probe may park the
// warp for a while, a span of the SM clock as well: about 0.2 s).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && clock64() - t0 > 400000000ll) return false;
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

// ---- element conversion ---------------------------------------------------------------------------------------
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
// acc += a.lo * b.lo + a.hi * b.hi for a packed pair of 16-bit floats, with the mixed-precision FMA of sm_100
// (f16/bf16 operands, f32 accumulator: the products are exact in f32, so this equals converting first).
template <typename T>
__device__ __forceinline__ void fma_pair(float& acc, uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ void fma_pair<__half>(float& acc, uint32_t a, uint32_t b) {
  asm("{\n"
      ".reg .b16 al, ah, bl, bh;\n"
      "mov.b32 {al, ah}, %1;\n"
      "mov.b32 {bl, bh}, %2;\n"
      "fma.rn.f32.f16 %0, al, bl, %0;\n"
      "fma.rn.f32.f16 %0, ah, bh, %0;\n"
      "}\n"
      : "+f"(acc)
      : "r"(a), "r"(b));
}
template <>
__device__ __forceinline__ void fma_pair<__nv_bfloat16>(float& acc, uint32_t a, uint32_t b) {
  asm("{\n"
      ".reg .b16 al, ah, bl, bh;\n"
      "mov.b32 {al, ah}, %1;\n"
      "mov.b32 {bl, bh}, %2;\n"
      "fma.rn.f32.bf16 %0, al, bl, %0;\n"
      "fma.rn.f32.bf16 %0, ah, bh, %0;\n"
      "}\n"
      : "+f"(acc)
      : "r"(a), "r"(b));
}
// acc += dot of two vectors of eight 16-bit floats
template <typename T>
__device__ __forceinline__ void dot8(float& acc, const uint4& a, const uint4& b) {
  fma_pair<T>(acc, a.x, b.x);
  fma_pair<T>(acc, a.y, b.y);
  fma_pair<T>(acc, a.z, b.z);
  fma_pair<T>(acc, a.w, b.w);
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

// Number of tiles the launch has to visit (exact for a plan, the slot count otherwise).
__device__ __forceinline__ int tile_count(const TileSrc& s) {
  return s.mode == MODE_PLAN ? min(s.plan[PH_NTILES], s.slots) : s.slots;
}

// Which tokens / adapter does tile `tile_idx` cover?  False when the slot holds no work (or fails a range check,
// in which case the status word records why).
__device__ __forceinline__ bool lookup_tile(const TileSrc& s, const Tables& tb, int tile_idx, TileInfo& t,
                                            int32_t* status) {
  if (s.mode == MODE_PLAN) {
    const int32_t* hdr = s.plan;
    // resolved tiles: the entry's token ids are fetched together with the header and the record
    t.xrcap = s.xrcap;
    t.xt = s.xoff > 0 ? s.plan + s.xoff + static_cast<int64_t>(tile_idx) * (kXtHead + 4 * s.xrcap) : nullptr;
    int4 k0 = make_int4(0, 0, 0, 0), k1 = k0;
    if (t.xt != nullptr) {
      k0 = reinterpret_cast<const int4*>(t.xt)[0];
      k1 = reinterpret_cast<const int4*>(t.xt)[1];
    }
    t.tok[0] = k0.x, t.tok[1] = k0.y, t.tok[2] = k0.z, t.tok[3] = k0.w;
    t.tok[4] = k1.x, t.tok[5] = k1.y, t.tok[6] = k1.z, t.tok[7] = k1.w;
    const int n_tiles = hdr[PH_NTILES], h_xoff = hdr[PH_XOFF], h_xrcap = hdr[PH_XRCAP];
    const int4* rec = reinterpret_cast<const int4*>(s.plan + PH_WORDS + kTileWords * tile_idx);
    const int4 r0 = rec[0];
    const int4 r1 = rec[1];
    if (tile_idx >= n_tiles) return false;
    t.adapter = r0.x;
    t.first = r0.y;
    t.n = r0.z;
    t.r = r0.w;
    t.loc_base = r1.x;
    t.perm = s.plan + PH_WORDS + kTileWords * hdr[PH_MAXTILES];
    // the entry counts when the plan holds resolved tiles where this launch expects them (same offset, same cap)
    t.xok = t.xt != nullptr && h_xoff == s.xoff && h_xrcap == s.xrcap && r1.z != 0;
    // big groups an eligible layout lets the tensor-core kernels serve are theirs (same predicate as mma_serves)
    if (s.seg_split > 0 && r1.y != 0 && tb.pool_stride % t.r == 0 && t.r <= s.mma_max_rows) return false;
    return t.n > 0 && t.r > 0;
  }
  int64_t adapter;
  t.perm = nullptr;
  t.xt = nullptr;
  t.xrcap = 0;
  t.xok = false;
  if (s.mode == MODE_TOKEN) {
    if (tile_idx >= s.T) return false;
    adapter = s.ids[tile_idx];
    t.first = tile_idx;
    t.n = 1;
  } else {
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
    adapter = s.ids[seg];
    t.first = static_cast<int>(first);
    t.n = static_cast<int>(n);
  }
  if (adapter < 0 || adapter >= tb.n_adapters) {
    set_status(status, SLORA_STATUS_BAD_ID);
    return false;
  }
  const int64_t r4 = tb.ranks4[adapter];
  const int64_t st = tb.start[adapter];
  if (r4 < 0 || st < 0 || st + r4 > tb.loc_len || r4 > (int64_t(1) << 20)) {
    set_status(status, SLORA_STATUS_BAD_TABLE);
    return false;
  }
  t.adapter = static_cast<int>(adapter);
  t.r = static_cast<int>(r4 >> 2);
  t.loc_base = st;
  // long segments of an adapter the tensor-core kernels can serve are theirs (same predicate as mma_serves)
  if (s.mode == MODE_SEGMENT && s.seg_split > 0 && s.seg_len[tile_idx / s.tiles_per_seg] >= s.seg_split &&
      t.r >= 8 && t.r <= 128 && t.r % 8 == 0 && tb.pool_stride % t.r == 0 && t.r <= s.mma_max_rows)
    return false;
  return t.r > 0;
}

// (callers that may see resolved tiles index with constants - unrolled loops - so that tok[] stays in registers)
__device__ __forceinline__ int tile_token(const TileInfo& t, int i) {
  if (t.xok) return t.tok[i];
  return t.perm ? t.perm[t.first + i] : t.first + i;
}
// Pool row of slot row `pr` (< the cap when there are resolved tiles) of projection `qkvo` of the tile's adapter, not
// range-checked.  With resolved tiles the entry is read whether or not it turns out to count: the load does not
// wait for the header and the record, and the table is only chased when the entry does not count.
__device__ __forceinline__ int64_t tile_loc(const TileInfo& t, const Tables& tb, int qkvo, int64_t pr) {
  if (t.xt != nullptr) {
    const int v = t.xt[kXtHead + qkvo * t.xrcap + static_cast<int>(min(pr, static_cast<int64_t>(t.xrcap - 1)))];
    if (t.xok) return v;
  }
  return tb.loc[t.loc_base + static_cast<int64_t>(t.r) * qkvo + pr];
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

// Exchange step of the expand butterfly over 8 per-lane partial sums (see expand_finish).
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

// LPO lanes (= r / 8) share one output, each holding the partial dot product over its 8 values of k, for the 8
// loads m = 0..7 of the warp.  After the butterfly lane l owns NV = max(1, 8 / LPO) complete outputs, those of
// loads m_base(l) + i, i < NV, where m_base takes 4, 2, 1 from lane bits 0, 1, 2 (as far as LPO uses them).
template <int LPO>
__device__ __forceinline__ void expand_butterfly(float (&v)[8], int lane) {
  if (LPO >= 2) exch<4>(v, lane, 1);
  if (LPO >= 4) exch<2>(v, lane, 2);
  if (LPO >= 8) exch<1>(v, lane, 4);
  if (LPO >= 16) v[0] += __shfl_xor_sync(0xffffffffu, v[0], 8);
}
template <int LPO>
__device__ __forceinline__ int expand_m_base(int lane) {
  int m = 0;
  if (LPO >= 2) m += (lane & 1) ? 4 : 0;
  if (LPO >= 4) m += (lane & 2) ? 2 : 0;
  if (LPO >= 8) m += (lane & 4) ? 1 : 0;
  return m;
}

}  // namespace slora
