// Multi-adapter LoRA shrink / expand for B200 (sm_100a): host-side dispatch and the C ABI.
//
// What is computed (the reference's math, slora/csrc/bgmv/bgmv_impl.cuh:15-149 and :153-208):
//   shrink: delta[t, j] = sum_k x[t, k] * A_a[j, k]                   j < r_a,  a = adapter of token t
//   expand: y[t, o]    += scale_a * sum_k delta[t, k] * B_a[o, k]     k < r_a
// with A_a / B_a read in place from the paged pool through the start / ranks4 / loc tables.
//
// Kernels: lora_plan.cuh groups a batch's tokens by adapter; lora_pipelined.cuh holds the persistent
// warp-specialised kernels used whenever the layout allows; lora_simple.cuh holds the one-CTA-per-item kernels that
// serve every other layout.  SLORA_KERNELS=simple|pipelined in the environment forces a choice (for A/B timing).
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "lora_common.cuh"
#include "lora_pipelined.cuh"
#include "lora_rope.cuh"
#include "lora_mma.cuh"
#include "lora_plan.cuh"
#include "lora_simple.cuh"
#include "pool_ops.cuh"

using namespace slora;

namespace {

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
// Tensor parallelism: turn the all-gathered intermediates [N][nproj][T][Rl] (rank g's columns are rank rows
// [g * rs, (g + 1) * rs) of the token's adapter, rs = its per-rank slot rows) into plain delta rows
// out[p][t][g * rs + j].  One CTA per (token, projection); columns at and beyond the adapter's rank are left alone.
template <typename T>
__global__ void tp_regroup_kernel(T* __restrict__ out, const T* __restrict__ in, const int64_t* __restrict__ ids,
                                  const int64_t* __restrict__ ranks4, int N, int Rl, int64_t tokens,
                                  int64_t part_stride, int64_t n_adapters) {
  const int64_t t = blockIdx.x;
  const int p = blockIdx.y;
  const int64_t a = ids[t];
  if (a < 0 || a >= n_adapters) return;
  int64_t rs = ranks4[a] >> 2;
  if (rs <= 0) return;
  if (rs > Rl) rs = Rl;
  const int R = N * Rl;
  const int64_t row = static_cast<int64_t>(p) * tokens + t;
  for (int idx = threadIdx.x; idx < N * Rl; idx += blockDim.x) {
    const int g = idx / Rl, j = idx - g * Rl;
    if (j < rs) out[row * R + g * rs + j] = in[g * part_stride + row * Rl + j];
  }
}

// Tensor parallelism, exchange over peer memory: every rank writes its columns of the intermediates straight into
// every rank's delta buffer (its own included) in the regrouped layout of tp_regroup_kernel, then tells every rank so
// with a flag; the last CTA of the launch then waits (for a bounded time) until every rank's flag for this exchange
// has arrived.  Replaces all-gather + regroup by one small kernel whose traffic is NVLink stores.
//   full[g]  : rank g's buffer [2][3][T][R], R = n_parts * part_width; the caller names the half (q,k,v calls use
//              half 0, o calls half 1)
//   flags[g] : rank g's int32 [2][n_parts]; flags[g][half][r] = n once rank r's columns of the n-th exchange on
//              that half have landed on rank g
//   seq_state: this rank's int32 [2]: exchanges completed per half; the kernel reads it, works on number
//              seq_state[half] + 1 and, when its wait is over, stores that number back.  Keeping the count on the
//              device lets a captured CUDA graph be replayed (a count passed as a kernel argument would be frozen).
// Two alternating halves suffice: a rank reaches its next exchange on half h only after every peer signalled the
// exchange on the other half in between, which a peer does after the kernels that read half h on it (its expand)
// have completed.
constexpr int kTpTokensPerCta = 16;
constexpr long long kTpWaitCycles = 4000000000ll;  // about 2 s: ranks drift by host-side jitter, not more
struct TpExchangeArgs {
  const void* local;  // [nproj][T][part_width], this rank's shrink output
  void* full[kTpMaxParts];
  int32_t* flags[kTpMaxParts];
  int32_t* counter;  // one zero-initialised int32 of this rank's memory (CTA arrival counter)
  int32_t* status;
  const int64_t* ids;
  const int64_t* ranks4;
  int my_part, n_parts, nproj, part_width;
  int64_t T, n_adapters;
  int64_t full_tokens;  // token rows per projection in a delta buffer (>= T)
  int32_t* seq_state;
  int half;
  int mode;  // bit 0: write and signal, bit 1: wait for every rank's signal, bit 2: the write is a plain block copy
             // of local [T][part_width] into slot my_part of every rank's [n_parts][full_tokens][part_width]
};

template <typename T>
__global__ void __launch_bounds__(128) tp_exchange_kernel(const TpExchangeArgs a) {
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int half = a.half;
  // under programmatic dependent launch the next kernel (the expand) may start now and fetch its adapter rows while
  // this exchange is in flight; this kernel itself needs the shrink's output, so it waits for the kernel before it
  pdl_launch_dependents();
  pdl_wait();
  // every CTA reads the count before the last one (which alone stores to it, at the very end) can get that far
  const int seq = a.seq_state[half] + 1;
  const int N = a.n_parts, pw = a.part_width;
  const int64_t R = static_cast<int64_t>(N) * pw;
  if ((a.mode & 5) == 5) {
    // partial sums travel unchanged: 16-byte copies of this rank's rows into its slot on every rank
    const int64_t vec_per_row = static_cast<int64_t>(pw) * sizeof(T) / 16;
    const int64_t total = a.T * vec_per_row;
    const uint4* src = reinterpret_cast<const uint4*>(a.local);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + tid; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const uint4 v = src[i];
      for (int g = 0; g < N; ++g)
        reinterpret_cast<uint4*>(a.full[g])[static_cast<int64_t>(a.my_part) * a.full_tokens * vec_per_row + i] = v;
    }
  } else if (a.mode & 1) {
    const int p = blockIdx.x % a.nproj;
    const int64_t t0 = static_cast<int64_t>(blockIdx.x / a.nproj) * kTpTokensPerCta;
    const T* local = reinterpret_cast<const T*>(a.local);
    for (int idx = tid; idx < kTpTokensPerCta * N * pw; idx += blockDim.x) {
      const int tt = idx / (N * pw);
      const int rem = idx - tt * (N * pw);
      const int g = rem / pw, j = rem - g * pw;
      const int64_t t = t0 + tt;
      if (t >= a.T) continue;
      const int64_t ad = a.ids[t];
      if (ad < 0 || ad >= a.n_adapters) continue;
      int64_t rs = a.ranks4[ad] >> 2;
      if (rs > pw) rs = pw;
      if (j >= rs) continue;
      T* dst = reinterpret_cast<T*>(a.full[g]) + ((static_cast<int64_t>(half) * 3 + p) * a.full_tokens + t) * R;
      dst[a.my_part * rs + j] = local[(static_cast<int64_t>(p) * a.T + t) * pw + j];
    }
  }
  // the last CTA to get here speaks for the launch
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int total = static_cast<int>(gridDim.x);
    s_last = atomicAdd(a.counter, 1) == total - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (tid == 0) *a.counter = 0;
  __threadfence_system();
  if ((a.mode & 1) && tid < N) {
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(a.flags[tid] + half * N + a.my_part), "r"(seq) : "memory");
  }
  if ((a.mode & 2) && tid < N) {
    const int32_t* mine = a.flags[a.my_part] + half * N + tid;
    const long long t_start = clock64();
    bool seen = false;
    while (!seen) {
      int v;
      asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      seen = v >= seq;
      if (!seen && clock64() - t_start > kTpWaitCycles) break;
    }
    if (!seen) set_status(a.status, SLORA_STATUS_TIMEOUT);
  }
  __threadfence_system();
  __syncthreads();
  if ((a.mode & 2) && tid == 0) a.seq_state[half] = seq;
}

// Adapter load: rows of one adapter for many layers and both buffers go into the pool in one launch.
// src[l] is the adapter's [2][n_rows][row_elems] block of layer l (A rows, then B rows); row i lands in pool row
// loc[i] of key_buffer[l] (A) and value_buffer[l] (B).  One CTA per (row, buffer, layer); 16-byte copies.
constexpr int kScatterLayers = 64;  // layers per launch (pointer tables travel as kernel arguments)
struct PoolScatterArgs {
  void* key[kScatterLayers];
  void* value[kScatterLayers];
  const void* src[kScatterLayers];
  const int64_t* loc;
  int64_t n_rows, row_bytes, pool_rows, pool_row_bytes;
  int n_layers;
  int32_t* status;
};
__global__ void __launch_bounds__(256) pool_scatter_kernel(const PoolScatterArgs a) {
  const int64_t i = blockIdx.x;
  const int which = blockIdx.y;  // 0: A rows -> key buffer, 1: B rows -> value buffer
  const int l = blockIdx.z;
  const int64_t row = a.loc[i];
  if (row < 0 || row >= a.pool_rows) {
    if (threadIdx.x == 0) set_status(a.status, SLORA_STATUS_BAD_TABLE);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(a.src[l]) +
                                                    (static_cast<int64_t>(which) * a.n_rows + i) * a.row_bytes);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(which == 0 ? a.key[l] : a.value[l]) + row * a.pool_row_bytes);
  for (int64_t c = threadIdx.x; c < a.row_bytes / 16; c += blockDim.x) dst[c] = src[c];
}

// out[i] = sum over ranks of parts[g][i], FP32 accumulation, i over T * width elements (width a multiple of 8).
template <typename T>
__global__ void __launch_bounds__(256) tp_sum_parts_kernel(T* __restrict__ out, const T* __restrict__ parts, int n_parts,
                                                           int64_t tokens, int64_t full_tokens, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t vec_per_row = width / 8;
  const int64_t total = tokens * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int g = 0; g < n_parts; ++g) {
      const uint4 v = reinterpret_cast<const uint4*>(parts)[static_cast<int64_t>(g) * full_tokens * vec_per_row + i];
      float f[8];
      cvt8<T>(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    union {
      uint4 q;
      T e[8];
    } pk;
#pragma unroll
    for (int e = 0; e < 8; ++e) pk.e[e] = from_f32<T>(acc[e]);
    reinterpret_cast<uint4*>(out)[i] = pk.q;
  }
}

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

// Kernels launched so far by this process, per family: 0 simple, 1 pipelined, 2 tensor core, 3 plan / tables.
std::atomic<long long> g_launches[4];

int check_launch(const char* what, int kernels) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  g_launches[3].fetch_add(kernels, std::memory_order_relaxed);
  return SLORA_OK;
}

int max_tiles_for(int64_t T, int64_t n_adapters) {
  const int64_t groups = T < n_adapters ? T : n_adapters;
  return static_cast<int>((T + kTileTokens - 1) / kTileTokens + groups);
}

// Big-tile slots a plan can need: a big group has c >= kBigGroupTokens tokens and ceil(c / 128) <= 2c / 128 tiles.
int max_big_for(int64_t T) { return static_cast<int>(2 * T / kBigGroupTokens + 1); }

struct PlanLayout {
  int max_tiles;
  int max_big;
  size_t words;
  int xoff;  // word offset of the resolved tiles (0: none)
};
// Rank cap of a plan's resolved tiles for a caller's max_rank: a multiple of 8 up to 128 (0: none).
int resolved_cap(int max_rank) {
  if (max_rank <= 0) return 0;
  const int cap = (max_rank + 7) & ~7;
  return cap > 128 ? 0 : cap;
}

PlanLayout plan_layout(int64_t T, int64_t n_adapters, int xrcap = 0) {
  PlanLayout l;
  l.max_tiles = max_tiles_for(T, n_adapters);
  l.max_big = max_big_for(T);
  l.words = static_cast<size_t>(PH_WORDS) + static_cast<size_t>(kTileWords) * l.max_tiles + 2u * static_cast<size_t>(T) +
            static_cast<size_t>(n_adapters) + 4 + static_cast<size_t>(kTileWords) * l.max_big;
  l.xoff = 0;
  if (xrcap > 0) {
    l.words = (l.words + 3) & ~static_cast<size_t>(3);
    if (l.words + static_cast<size_t>(l.max_tiles) * (kXtHead + 4 * xrcap) < 0x7fffffffu) {
      l.xoff = static_cast<int>(l.words);
      l.words += static_cast<size_t>(l.max_tiles) * (kXtHead + 4 * xrcap);
    }
  }
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

// Which kernel family serves a call: the pipelined kernels when the layout allows, unless the environment says
// otherwise.
enum KernelChoice { CHOOSE_AUTO = 0, CHOOSE_SIMPLE = 1, CHOOSE_PIPELINED = 2 };
KernelChoice kernel_choice() {
  static const KernelChoice choice = [] {
    const char* e = getenv("SLORA_KERNELS");
    if (e && strcmp(e, "simple") == 0) return CHOOSE_SIMPLE;
    if (e && strcmp(e, "pipelined") == 0) return CHOOSE_PIPELINED;
    return CHOOSE_AUTO;
  }();
  return choice;
}

// The tensor-core kernels for long segments can be switched off with SLORA_MMA=0.
bool mma_enabled() {
  static const bool on = [] {
    const char* e = getenv("SLORA_MMA");
    return !(e && strcmp(e, "0") == 0);
  }();
  return on && kernel_choice() != CHOOSE_SIMPLE;
}

int sm_count() {
  static int count[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    count[dev] = n;
  }
  return count[dev];
}

int family_of(const char* what) {
  if (strstr(what, "tp_exchange")) return 3;
  if (strstr(what, "tensor core")) return 2;
  if (strstr(what, "pipelined")) return 1;
  return 0;
}

template <typename K, typename A>
int launch(K kernel, int64_t grid, int threads, size_t smem, unsigned flags, cudaStream_t stream, const A& args,
           const char* what) {
  if (grid <= 0) return SLORA_OK;
  if (grid > 0x7fffffffLL) return fail(SLORA_ERR_SHAPE, "%s: grid of %lld CTAs is too large", what, (long long)grid);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
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
  g_launches[family_of(what)].fetch_add(1, std::memory_order_relaxed);
  return SLORA_OK;
}

// A call that launches a tensor-core kernel and a CUDA-core kernel runs the two side by side: they work on disjoint
// tokens, so the tensor-core kernel goes to a library-owned side stream that forks from the caller's stream before
// the launch and joins it again after the CUDA-core launch (also under stream capture, where the pair becomes two
// parallel branches of the graph).  One side stream and two events per device, created at first use and kept.
// SLORA_SIDE_STREAM=0 keeps everything on the caller's stream.
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join;
  int state;  // 0 = not created yet, 1 = usable, -1 = creation failed or switched off
};
SideStream* side_stream() {
  static SideStream sides[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return nullptr;
  }
  SideStream& sd = sides[dev];
  if (sd.state == 0) {
    const char* e = getenv("SLORA_SIDE_STREAM");
    sd.state = -1;
    if (!(e && strcmp(e, "0") == 0) &&
        cudaStreamCreateWithFlags(&sd.stream, cudaStreamNonBlocking) == cudaSuccess &&
        cudaEventCreateWithFlags(&sd.fork, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventCreateWithFlags(&sd.join, cudaEventDisableTiming) == cudaSuccess) {
      sd.state = 1;
    } else {
      cudaGetLastError();
    }
  }
  return sd.state == 1 ? &sd : nullptr;
}
// Fork: returns the stream the tensor-core kernel should use (the side stream, or `main` when there is none).
cudaStream_t fork_side(SideStream* sd, cudaStream_t main) {
  if (!sd) return main;
  if (cudaEventRecord(sd->fork, main) != cudaSuccess || cudaStreamWaitEvent(sd->stream, sd->fork, 0) != cudaSuccess) {
    cudaGetLastError();
    return main;
  }
  return sd->stream;
}
// Join on scope exit: whatever the caller's stream does next waits for the side stream's work of this call.
struct SideJoin {
  SideStream* sd = nullptr;
  cudaStream_t main = nullptr;
  void arm(SideStream* s, cudaStream_t m) {
    if (cudaEventRecord(s->join, s->stream) == cudaSuccess) {
      sd = s;
      main = m;
    } else {
      cudaGetLastError();
    }
  }
  ~SideJoin() {
    if (sd && cudaStreamWaitEvent(main, sd->join, 0) != cudaSuccess) cudaGetLastError();
  }
};

// The same with a second kernel argument (a tensor map or a set of them).
template <typename K, typename A, typename B>
int launch2(K kernel, int64_t grid, int threads, size_t smem, unsigned flags, cudaStream_t stream, const A& args,
            const B& extra, const char* what, int cluster = 1) {
  if (grid <= 0) return SLORA_OK;
  if (grid > 0x7fffffffLL) return fail(SLORA_ERR_SHAPE, "%s: grid of %lld CTAs is too large", what, (long long)grid);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (flags & SLORA_FLAG_PDL) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (cluster > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args, extra);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  g_launches[family_of(what)].fetch_add(1, std::memory_order_relaxed);
  return SLORA_OK;
}

// 2-D tensor map over a row-major [rows x inner] matrix of 16-bit elements with a box of [box_rows x 64] elements
// and the 128-byte swizzle (the layout tcgen05.mma and the TMA reduce of the tensor-core kernels expect).  The
// driver's encoder is looked up once through the runtime, so the library does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int make_tmap(CUtensorMap* map, int dtype, const void* base, int64_t inner, int64_t rows, int64_t row_stride_elems,
              int box_rows) {
  static EncodeTiledFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      fn = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
  }();
  if (!encode) return fail(SLORA_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride_elems) * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, dtype == SLORA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                            2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SLORA_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return SLORA_OK;
}

// Opt in to more than 48 KB of dynamic shared memory, once per (kernel, device) and size high-water mark.
// (Kernels with sizeable static shared memory pass static_bytes: the 48 KB default limit covers both kinds.)
template <typename K>
int ensure_dyn_smem(K kernel, int which, size_t smem, size_t static_bytes = 0) {
  static int high_water[16][64];  // one row per kernel template (`which`)
  if (smem + static_bytes <= 48 * 1024) return SLORA_OK;
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

// Grid of a pipelined launch: two CTAs per SM, or one per item when there are fewer.  Under the padded enumeration
// (slot i belongs to CTA i mod grid, `per_tile` slots per tile) the grid is made coprime to per_tile: with a common
// factor a CTA only ever sees some of a tile's slot kinds, and where low-rank adapters leave the same kinds empty
// every time (the second row block of a projection, say) the CTAs that see those would idle while the others do all
// the work - e.g. 296 CTAs and 6 slots per tile: the odd CTAs would only get second row blocks.
// Off unless SLORA_COPRIME_GRID=1: measured on one GPU only (a rank's kernels of the 13B-shaped batch under 8-way
// tensor parallelism, emulated: 54.1 -> 51.6 us per layer; same-rank decode batches unchanged).
int64_t pipe_grid(int64_t items, int per_tile, bool exact) {
  static const bool coprime = [] {
    const char* e = getenv("SLORA_COPRIME_GRID");
    return e && strcmp(e, "1") == 0;
  }();
  int64_t grid = static_cast<int64_t>(sm_count()) * kPipeCtasPerSm;
  if (items < grid) return items;
  if (coprime && !exact && per_tile > 1) {
    auto gcd = [](int64_t a, int64_t b) {
      while (b) {
        const int64_t t = a % b;
        a = b;
        b = t;
      }
      return a;
    };
    while (grid > 1 && gcd(grid, per_tile) != 1) --grid;
  }
  return grid;
}

int run_shrink(const TileSrc& src, const Tables& tb, const void* w, const void* x, int64_t x_stride, int h_in,
               int nproj, const int* qkvo, void* const* delta, int64_t delta_stride, int delta_width, int dtype,
               unsigned flags, int32_t* status, cudaStream_t stream, const TpLink* tp = nullptr, int rank_mult = 1) {
  int rc = check_common(dtype, tb, w);
  if (rc) return rc;
  if (rank_mult < 1) return fail(SLORA_ERR_SHAPE, "rank_mult must be >= 1");
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
  a.src.xoff = a.src.xrcap = 0;  // resolved tiles are the pipelined kernels' (set where those are launched)
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
  a.rank_mult = rank_mult;
  a.status = status;
  // long segments first go to the tensor-core kernel; the launch below then skips them
  a.src.seg_split = 0;
  SideJoin side_join;
  if (tp) {
    a.tp = *tp;
    a.tp.enabled = 1;
  }
  if (!tp && rank_mult == 1 && (src.mode == MODE_SEGMENT || src.mode == MODE_PLAN) && src.seg_split > 0 &&
      mma_enabled() && S == h_in &&
      h_in % kMmaKBlock == 0 && src.T < 0x7fffffff) {
    bool consecutive = true;
    for (int p = 1; p < nproj; ++p) consecutive = consecutive && qkvo[p] == qkvo[0] + p;
    const int wmax = delta_width < kMmaMaxRank ? delta_width : kMmaMaxRank;
    const int gp = (consecutive && nproj * wmax <= kMmaMaxRows) ? nproj : 1;
    const int npad_max = (gp * wmax + 15) & ~15;
    ShrinkArgs m = a;
    m.src.seg_split = src.seg_split;
    m.src.mma_max_rows = wmax;
    m.rows_per_cta = gp;
    m.max_rb = nproj / gp;
    m.mma_stage_bytes = kMmaXTileBytes + npad_max * kMmaKBlock * 2;
    const int64_t mma_tiles = src.mode == MODE_PLAN ? src.big_slots : static_cast<int64_t>(src.n_seg) * src.mma_tiles_per_seg;
    // split K over a cluster of up to 8 CTAs while the launch would otherwise leave SMs idle (a tile alone streams
    // 128 x h_in activations through one SM); a plan enumerates about twice the tiles it can hold
    // (when the caller passed the plan's own count of big tiles, SLORA_FLAG_BIG_TILES, big_slots is exact)
    const int64_t likely_units =
        (src.mode == MODE_PLAN ? (src.big_exact ? mma_tiles : src.T / kBigTileTokens + 1) : mma_tiles) * m.max_rb;
    const int nkb_total = h_in / kMmaKBlock;
    // clusters are placed inside one GPC (about 18 SMs): of size 8 two fit a GPC, of size 4 four - a launch that
    // wants more clusters than fit at once runs in waves, each as long as the whole K loop of a CTA
    auto fits_one_wave = [&](int k) {
      const int clusters_at_once = k >= 8 ? sm_count() / 9 : (k == 4 ? sm_count() / 9 * 2 : sm_count() / k);
      return likely_units <= clusters_at_once;
    };
    int ks = 8;
    while (ks > 1 && (nkb_total % ks != 0 || !fits_one_wave(ks))) ks >>= 1;
    m.mma_ksplit = ks;
    m.mma_stages = (kMmaSmemBudget - 1024) / m.mma_stage_bytes;
    if (m.mma_stages > kMmaMaxStages) m.mma_stages = kMmaMaxStages;
    if (m.mma_stages > nkb_total / ks) m.mma_stages = nkb_total / ks;
    size_t smem = static_cast<size_t>(m.mma_stages) * m.mma_stage_bytes;
    const size_t red_bytes = static_cast<size_t>(kMmaTokens) * (npad_max + 4) * 4;  // split-K partial sums
    if (ks > 1 && smem < red_bytes) smem = red_bytes;
    smem += 1024;
    // Tensor memory: a CTA takes 128 or 256 of the SM's 512 columns and tcgen05.alloc blocks while they are taken.
    // CTAs of two clusters blocked on each other's columns would never reach their cluster barriers, so the
    // shared-memory request is kept large enough that the CTAs that fit on an SM never want more than 512 columns.
    const size_t min_smem = (npad_max > 128 ? 80 : 48) * 1024;
    if (smem < min_smem) smem = min_smem;
    const int64_t grid = mma_tiles * m.max_rb * ks;
    CUtensorMap x_map;
    rc = make_tmap(&x_map, dtype, x, h_in, src.T, x_stride, kMmaTokens);
    if (rc) return rc;
    // (calls chained with programmatic dependent launch stay on one stream: measured, the chain's overlap is worth
    // more than running the pair side by side)
    SideStream* sd = (flags & SLORA_FLAG_PDL) ? nullptr : side_stream();
    const cudaStream_t mma_stream = fork_side(sd, stream);
    if (dtype == SLORA_F16) {
      auto k = lora_shrink_mma_kernel<__half>;
      rc = ensure_dyn_smem(k, 4, smem, 4096);
      if (!rc) rc = launch2(k, grid, kMmaShrinkThreads, smem, flags, mma_stream, m, x_map, "shrink(tensor core)", ks);
    } else {
      auto k = lora_shrink_mma_kernel<__nv_bfloat16>;
      rc = ensure_dyn_smem(k, 5, smem, 4096);
      if (!rc) rc = launch2(k, grid, kMmaShrinkThreads, smem, flags, mma_stream, m, x_map, "shrink(tensor core)", ks);
    }
    if (mma_stream != stream) side_join.arm(sd, stream);
    if (rc) return rc;
    // every group of the plan is a big group the tensor-core launch serves: nothing is left for the CUDA cores
    if ((flags & SLORA_FLAG_ONLY_BIG) && src.mode == MODE_PLAN) return SLORA_OK;
    a.src.seg_split = src.seg_split;
    a.src.mma_max_rows = wmax;
    // without a side stream the CUDA-core launch of the same call may still start while the tensor-core kernel
    // runs: neither writes what the other reads before its grid-dependency wait, and their outputs are disjoint
    if (mma_stream == stream) flags |= SLORA_FLAG_PDL;
  }
  const bool can_pipe = (S % h_in == 0);
  const KernelChoice choice = kernel_choice();
  if ((choice == CHOOSE_PIPELINED || tp) && !can_pipe)
    return fail(SLORA_ERR_SHAPE, "No suitable kernel. pipelined shrink needs pool_stride %% h_in == 0");
  if (tp && choice == CHOOSE_SIMPLE) return fail(SLORA_ERR_SHAPE, "No suitable kernel. the linked shrink is pipelined only");
  if (can_pipe && choice != CHOOSE_SIMPLE) {
    a.rows_per_cta = kMaxRows;
    a.src.xoff = src.xoff;
    a.src.xrcap = src.xrcap;
    a.max_rb = (delta_width + kMaxRows - 1) / kMaxRows;
    const int64_t items = static_cast<int64_t>(src.slots) * nproj * a.max_rb;
    const bool exact = (flags & SLORA_FLAG_EXACT_ITEMS) != 0 && src.mode == MODE_PLAN;
    const int64_t grid = pipe_grid(items, nproj * a.max_rb, exact);
    const size_t smem = kRingBytes;
    auto go = [&](auto k, int which) {
      const int rc2 = ensure_dyn_smem(k, which, smem);
      return rc2 ? rc2 : launch(k, grid, kPipeThreads, smem, flags, stream, a, "shrink(pipelined)");
    };
    if (dtype == SLORA_F16) return exact ? go(lora_shrink_pipe_kernel<__half, true>, 4) : go(lora_shrink_pipe_kernel<__half, false>, 2);
    return exact ? go(lora_shrink_pipe_kernel<__nv_bfloat16, true>, 5) : go(lora_shrink_pipe_kernel<__nv_bfloat16, false>, 3);
  }
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
  const int64_t grid = static_cast<int64_t>(src.slots) * nproj * a.max_rb;
  if (dtype == SLORA_F16) {
    auto k = lora_shrink_kernel<__half>;
    rc = ensure_dyn_smem(k, 0, smem);
    return rc ? rc : launch(k, grid, kThreads, smem, flags, stream, a, "shrink");
  }
  auto k = lora_shrink_kernel<__nv_bfloat16>;
  rc = ensure_dyn_smem(k, 1, smem);
  return rc ? rc : launch(k, grid, kThreads, smem, flags, stream, a, "shrink");
}

int run_expand(const TileSrc& src, const Tables& tb, const void* w, const void* scales, int nproj, const int* qkvo,
               void* const* y, const int64_t* y_stride, const int* h_out, const void* const* delta,
               int64_t delta_stride, int delta_width, int delta_parts, int64_t delta_part_stride, int rank_mult,
               int dtype, unsigned flags, int32_t* status, cudaStream_t stream, const TpLink* tp = nullptr,
               const RopeArgs* epi = nullptr) {
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
  a.src.xoff = a.src.xrcap = 0;  // resolved tiles are the pipelined kernels' (set where those are launched)
  a.tb = tb;
  a.w = w;
  a.scales = scales;
  a.nproj = nproj;
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
  }
  // work items per (tile, projection): chunks of `chunk` flat B elements at the widest rank the delta can hold
  auto set_chunks = [&](int chunk) {
    a.chunk_begin[0] = 0;
    for (int p = 0; p < nproj; ++p) {
      const int64_t chunks = (static_cast<int64_t>(h_out[p]) * max_rank + chunk - 1) / chunk;
      a.chunk_begin[p + 1] = a.chunk_begin[p] + static_cast<int>(chunks);
    }
  };
  a.delta_stride = delta_stride;
  a.delta_parts = delta_parts;
  a.delta_part_stride = delta_part_stride;
  a.rank_mult = rank_mult;
  a.max_rank = max_rank;
  a.status = status;
  a.src.seg_split = 0;
  SideJoin side_join;
  if (tp) {
    a.tp = *tp;
    a.tp.enabled = 1;
  }
  bool can_mma = !tp && !epi && (src.mode == MODE_SEGMENT || src.mode == MODE_PLAN) && src.seg_split > 0 &&
                 mma_enabled() && delta_parts == 1 && rank_mult == 1 && delta_stride % 8 == 0;
  for (int p = 0; p < nproj; ++p)
    can_mma = can_mma && aligned16(y[p]) && y_stride[p] % 8 == 0 && aligned16(delta[p]);
  for (int p = 0; p < nproj; ++p) can_mma = can_mma && h_out[p] >= 64;
  can_mma = can_mma && tb.pool_stride < 0x7fffffff && src.T < 0x7fffffff;
  if (can_mma) {
    ExpandArgs m = a;
    m.src.seg_split = src.seg_split;
    m.src.mma_max_rows = delta_width < kMmaMaxRank ? delta_width : kMmaMaxRank;
    m.chunk_begin[0] = 0;
    for (int p = 0; p < nproj; ++p)
      m.chunk_begin[p + 1] = m.chunk_begin[p] + (h_out[p] + kMmaOutPerCta - 1) / kMmaOutPerCta;
    const int wmax = delta_width < kMmaMaxRank ? delta_width : kMmaMaxRank;
    m.mma_stage_bytes = kMmaTokens * ((wmax + 15) & ~15) * 2;
    const size_t smem = kMmaOutTileBytes + static_cast<size_t>(1 + kMmaExStages) * m.mma_stage_bytes + 1024;
    const int64_t mma_tiles = src.mode == MODE_PLAN ? src.big_slots : static_cast<int64_t>(src.n_seg) * src.mma_tiles_per_seg;
    const int64_t grid = mma_tiles * m.chunk_begin[nproj];
    TmapSet y_maps;
    memset(&y_maps, 0, sizeof(y_maps));
    for (int p = 0; p < nproj && !rc; ++p)
      rc = make_tmap(&y_maps.m[p], dtype, y[p], h_out[p], src.T, y_stride[p], kMmaTokens);
    if (rc) return rc;
    // (calls chained with programmatic dependent launch stay on one stream: measured, the chain's overlap is worth
    // more than running the pair side by side)
    SideStream* sd = (flags & SLORA_FLAG_PDL) ? nullptr : side_stream();
    const cudaStream_t mma_stream = fork_side(sd, stream);
    if (dtype == SLORA_F16) {
      auto k = lora_expand_mma_kernel<__half>;
      rc = ensure_dyn_smem(k, 6, smem, 12288);
      if (!rc) rc = launch2(k, grid, kMmaExpandThreads, smem, flags, mma_stream, m, y_maps, "expand(tensor core)");
    } else {
      auto k = lora_expand_mma_kernel<__nv_bfloat16>;
      rc = ensure_dyn_smem(k, 7, smem, 12288);
      if (!rc) rc = launch2(k, grid, kMmaExpandThreads, smem, flags, mma_stream, m, y_maps, "expand(tensor core)");
    }
    if (mma_stream != stream) side_join.arm(sd, stream);
    if (rc) return rc;
    if ((flags & SLORA_FLAG_ONLY_BIG) && src.mode == MODE_PLAN) return SLORA_OK;  // as in the shrink
    a.src.seg_split = src.seg_split;
    a.src.mma_max_rows = delta_width < kMmaMaxRank ? delta_width : kMmaMaxRank;
    if (mma_stream == stream) flags |= SLORA_FLAG_PDL;  // as in the shrink
  }
  const int pipe_piece = pow2_divisor(tb.pool_stride, kPipeChunk);
  bool can_pipe = delta_parts == 1 && delta_stride % 8 == 0 && pipe_piece * kMaxPieces >= kPipeChunk &&
                  tb.pool_stride < (int64_t(1) << 30) &&
                  (kPipeChunk - 1) / tb.pool_stride + 2 <= kSpanRows;
  for (int p = 0; p < nproj; ++p)
    can_pipe = can_pipe && aligned16(y[p]) && y_stride[p] % 8 == 0 && aligned16(delta[p]);
  const KernelChoice choice = kernel_choice();
  if ((choice == CHOOSE_PIPELINED || tp) && !can_pipe)
    return fail(SLORA_ERR_ALIGN, "No suitable kernel. pipelined expand needs 16-byte aligned y and delta rows and a "
                                 "plain delta layout");
  if (tp && choice == CHOOSE_SIMPLE) return fail(SLORA_ERR_SHAPE, "No suitable kernel. the linked expand is pipelined only");
  if (can_pipe && choice != CHOOSE_SIMPLE) {
    a.piece = pipe_piece;
    a.src.xoff = src.xoff;
    a.src.xrcap = src.xrcap;
    set_chunks(kPipeChunk);
    const int64_t items = static_cast<int64_t>(src.slots) * a.chunk_begin[nproj];
    const bool exact = (flags & SLORA_FLAG_EXACT_ITEMS) != 0 && src.mode == MODE_PLAN;
    const int64_t grid = pipe_grid(items, a.chunk_begin[nproj], exact);
    const size_t smem = exact ? kExpandRingBytes : kRingBytes;
    if (epi) {
      // the expand with rotary embedding / KV-pool scatter in its epilogue (lora_rope.cuh)
      auto go2 = [&](auto k, int which) {
        const int rc2 = ensure_dyn_smem(k, which, smem);
        return rc2 ? rc2 : launch2(k, grid, kPipeThreads, smem, flags, stream, a, *epi, "expand(pipelined, rotary)");
      };
      if (dtype == SLORA_F16) return exact ? go2(lora_expand_rope_pipe_kernel<__half, true>, 2) : go2(lora_expand_rope_pipe_kernel<__half, false>, 0);
      return exact ? go2(lora_expand_rope_pipe_kernel<__nv_bfloat16, true>, 3) : go2(lora_expand_rope_pipe_kernel<__nv_bfloat16, false>, 1);
    }
    auto go = [&](auto k, int which) {
      const int rc2 = ensure_dyn_smem(k, which, smem);
      return rc2 ? rc2 : launch(k, grid, kPipeThreads, smem, flags, stream, a, "expand(pipelined)");
    };
    if (tp && tp->inband) {  // the instantiation that checks whether the delta values have arrived
      if (dtype == SLORA_F16)
        return exact ? go(lora_expand_pipe_kernel<__half, true, true>, 12) : go(lora_expand_pipe_kernel<__half, false, true>, 10);
      return exact ? go(lora_expand_pipe_kernel<__nv_bfloat16, true, true>, 13)
                   : go(lora_expand_pipe_kernel<__nv_bfloat16, false, true>, 11);
    }
    if (dtype == SLORA_F16) return exact ? go(lora_expand_pipe_kernel<__half, true>, 4) : go(lora_expand_pipe_kernel<__half, false>, 2);
    return exact ? go(lora_expand_pipe_kernel<__nv_bfloat16, true>, 5) : go(lora_expand_pipe_kernel<__nv_bfloat16, false>, 3);
  }
  if (epi) return fail(SLORA_ERR_SHAPE, "No suitable kernel. the expand with a rotary epilogue is pipelined only");
  a.piece = piece;
  set_chunks(kChunk);
  const int64_t grid = static_cast<int64_t>(src.slots) * a.chunk_begin[nproj];
  if (dtype == SLORA_F16) return launch(lora_expand_kernel<__half>, grid, kThreads, 0, flags, stream, a, "expand");
  return launch(lora_expand_kernel<__nv_bfloat16>, grid, kThreads, 0, flags, stream, a, "expand");
}

int make_src(const void* plan, const int64_t* ids, int64_t T, int64_t n_adapters, unsigned flags, TileSrc* src,
             int32_t** status) {
  memset(src, 0, sizeof(*src));
  src->T = T;
  *status = nullptr;
  if (T < 0 || T > 0x3fffffff) return fail(SLORA_ERR_SHAPE, "T=%lld out of range", (long long)T);
  if (plan) {
    if (!aligned16(plan)) return fail(SLORA_ERR_ALIGN, "plan workspace is not 16-byte aligned");
    src->mode = MODE_PLAN;
    src->plan = reinterpret_cast<const int32_t*>(plan);
    src->slots = max_tiles_for(T, n_adapters);
    src->big_slots = max_big_for(T);
    // the caller read the plan's count of big tiles and passed it on: enumerate exactly those
    const int hint = static_cast<int>(flags >> 16);
    if (hint > 0 && hint <= src->big_slots) {
      src->big_slots = hint;
      src->big_exact = 1;
    }
    src->seg_split = ((flags & SLORA_FLAG_BIG_GROUPS) && T >= kBigGroupTokens) ? kBigGroupTokens : 0;
    // the caller says the plan was built with resolved tiles (SLORA_FLAG_RESOLVED): where the launch will look
    const int cap = static_cast<int>((flags >> 8) & 0x1fu) * 8;
    if (cap > 0 && cap <= 128) {
      src->xoff = plan_layout(T, n_adapters, cap).xoff;
      src->xrcap = src->xoff > 0 ? cap : 0;
    }
    *status = const_cast<int32_t*>(src->plan) + PH_STATUS;
  } else {
    if (!ids && T > 0) return fail(SLORA_ERR_NULL, "neither plan nor ids given");
    src->mode = MODE_TOKEN;
    src->ids = ids;
    src->slots = static_cast<int>(T);
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
  src->mma_tiles_per_seg = (max_seg_len + kMmaTokens - 1) / kMmaTokens;
  src->seg_split = max_seg_len >= kMmaMinTokens ? kMmaMinTokens : 0;
  src->T = (n_seg == 0 || src->tiles_per_seg == 0) ? 0 : T;
  if (static_cast<int64_t>(n_seg) * src->tiles_per_seg > 0x3fffffff)
    return fail(SLORA_ERR_SHAPE, "too many segment tiles");
  src->slots = n_seg * src->tiles_per_seg;
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

int slora_version(void) { return 103; }


void slora_launch_counts(int64_t out[4]) {
  for (int i = 0; i < 4; ++i) out[i] = g_launches[i].load(std::memory_order_relaxed);
}

const char* slora_last_error(void) { return g_err; }

int slora_bgmv_shrink(void* delta, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                      const int64_t* loc, const int64_t* ids, int qkvo, int64_t T, int h_in, int64_t x_stride,
                      int64_t delta_stride, int delta_width, int64_t pool_rows, int64_t pool_stride,
                      int64_t n_adapters, int64_t loc_len, int dtype, void* stream) {
  TileSrc src;
  int32_t* status;
  int rc = make_src(nullptr, ids, T, n_adapters, 0, &src, &status);
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
  int rc = make_src(nullptr, ids, T, n_adapters, 0, &src, &status);
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

size_t slora_plan_workspace_bytes(int64_t T, int64_t n_adapters) { return slora_plan_workspace_bytes_ex(T, n_adapters, 0); }

size_t slora_plan_workspace_bytes_ex(int64_t T, int64_t n_adapters, int max_rank) {
  if (T < 0 || n_adapters < 0) return 0;
  return plan_layout(T, n_adapters, resolved_cap(max_rank)).words * sizeof(int32_t);
}

int slora_plan_build(void* workspace, size_t workspace_bytes, const int64_t* ids, int64_t T, const int64_t* start,
                     const int64_t* ranks4, int64_t n_adapters, int64_t loc_len, void* stream) {
  return slora_plan_build_ex(workspace, workspace_bytes, ids, T, start, ranks4, nullptr, nullptr, n_adapters, loc_len, 0,
                             stream);
}

int slora_plan_build_ex(void* workspace, size_t workspace_bytes, const int64_t* ids, int64_t T, const int64_t* start,
                        const int64_t* ranks4, const int64_t* loc, const void* scales, int64_t n_adapters,
                        int64_t loc_len, int max_rank, void* stream) {
  if (!workspace || (!ids && T > 0)) return fail(SLORA_ERR_NULL, "workspace or ids is null");
  if (!start || !ranks4) return fail(SLORA_ERR_NULL, "start or ranks4 is null");
  if (!aligned16(workspace)) return fail(SLORA_ERR_ALIGN, "plan workspace is not 16-byte aligned");
  if (T < 0 || T > 0x3fffffff || n_adapters < 0 || n_adapters > 0x3fffffff)
    return fail(SLORA_ERR_SHAPE, "T=%lld or n_adapters=%lld out of range", (long long)T, (long long)n_adapters);
  const int cap = loc ? resolved_cap(max_rank) : 0;
  const PlanLayout l = plan_layout(T, n_adapters, cap);
  if (workspace_bytes < l.words * sizeof(int32_t))
    return fail(SLORA_ERR_WORKSPACE, "plan workspace has %zu bytes, needs %zu", workspace_bytes,
                l.words * sizeof(int32_t));
  plan_build_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<int32_t*>(workspace), ids, start, ranks4, loc_len, static_cast<int>(T),
      static_cast<int>(n_adapters), l.max_tiles, l.max_big, loc, static_cast<const unsigned short*>(scales), l.xoff,
      cap);
  plan_fence_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
  return check_launch("plan_build", 2);
}

int slora_plan_big_tiles(const void* workspace, int* n_big_out, void* stream) {
  if (!workspace || !n_big_out) return fail(SLORA_ERR_NULL, "workspace or n_big_out is null");
  int32_t hdr[PH_WORDS];
  cudaError_t e = cudaMemcpyAsync(hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "plan_big_tiles: %s", cudaGetErrorString(e));
  if (hdr[PH_MAGIC] != kPlanMagic) return fail(SLORA_ERR_WORKSPACE, "workspace does not hold a plan");
  *n_big_out = hdr[PH_NBIG];
  return SLORA_OK;
}

int slora_plan_info(const void* workspace, int* n_tiles_out, int* n_big_out, int* uniform_rank_out, void* stream) {
  if (!workspace) return fail(SLORA_ERR_NULL, "workspace is null");
  int32_t hdr[PH_WORDS];
  cudaError_t e = cudaMemcpyAsync(hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "plan_info: %s", cudaGetErrorString(e));
  if (hdr[PH_MAGIC] != kPlanMagic) return fail(SLORA_ERR_WORKSPACE, "workspace does not hold a plan");
  if (n_tiles_out) *n_tiles_out = hdr[PH_NTILES];
  if (n_big_out) *n_big_out = hdr[PH_NBIG];
  if (uniform_rank_out) *uniform_rank_out = hdr[PH_UNIFORM];
  return SLORA_OK;
}

int slora_plan_header(const void* workspace, int32_t out[16], void* stream) {
  if (!workspace || !out) return fail(SLORA_ERR_NULL, "workspace or out is null");
  cudaError_t e = cudaMemcpyAsync(out, workspace, PH_WORDS * sizeof(int32_t), cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "plan_header: %s", cudaGetErrorString(e));
  if (out[PH_MAGIC] != kPlanMagic) return fail(SLORA_ERR_WORKSPACE, "workspace does not hold a plan");
  return SLORA_OK;
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
  int rc = make_src(plan, ids, T, n_adapters, flags, &src, &status);
  if (rc) return rc;
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_a, x,
                    x_stride, h_in, nproj, qkvo, delta, delta_stride, delta_width, dtype, flags, status,
                    static_cast<cudaStream_t>(stream));
}

int slora_lora_shrink_rows(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* delta,
                           int64_t delta_stride, int delta_width, int rank_mult, const void* x, int64_t x_stride,
                           int h_in, const void* pool_a, int64_t pool_rows, int64_t pool_stride, const int64_t* start,
                           const int64_t* ranks4, const int64_t* loc, int64_t n_adapters, int64_t loc_len, int64_t T,
                           int dtype, unsigned flags, void* stream) {
  if (!qkvo || !delta) return fail(SLORA_ERR_NULL, "qkvo or delta array is null");
  TileSrc src;
  int32_t* status;
  int rc = make_src(plan, ids, T, n_adapters, flags, &src, &status);
  if (rc) return rc;
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_a, x,
                    x_stride, h_in, nproj, qkvo, delta, delta_stride, delta_width, dtype, flags, status,
                    static_cast<cudaStream_t>(stream), nullptr, rank_mult);
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
  int rc = make_src(plan, ids, T, n_adapters, flags, &src, &status);
  if (rc) return rc;
  return run_expand(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_b,
                    scales, nproj, qkvo, y, y_stride, h_out, delta, delta_stride, delta_width, delta_parts,
                    delta_part_stride, rank_mult, dtype, flags, status, static_cast<cudaStream_t>(stream));
}

int slora_tp_allsum(const void* local, void* const* peer_parts, int32_t* const* peer_flags, int32_t* counter,
                    int32_t* status, void* out, int my_part, int n_parts, int64_t T, int64_t full_tokens, int width,
                    int half, int32_t* seq_state, int mode, int dtype, unsigned flags, void* stream) {
  if (T == 0) return SLORA_OK;
  if ((mode & 3) == 0) return fail(SLORA_ERR_SHAPE, "tp_allsum: mode must hold 1 (write and signal) and/or 2 (wait, sum)");
  if (dtype != SLORA_F16 && dtype != SLORA_BF16) return fail(SLORA_ERR_DTYPE, "unsupported dtype %d", dtype);
  if (!local || !peer_parts || !peer_flags || !counter || !seq_state || !out) return fail(SLORA_ERR_NULL, "null argument");
  if (n_parts < 1 || n_parts > kTpMaxParts || my_part < 0 || my_part >= n_parts || half < 0 || half > 1 || T < 0 ||
      full_tokens < T || width < 8 || width % 8 != 0)
    return fail(SLORA_ERR_SHAPE, "tp_allsum: bad part, half, width (a multiple of 8) or buffer size");
  if (!aligned16(local) || !aligned16(out)) return fail(SLORA_ERR_ALIGN, "tp_allsum: buffers must be 16-byte aligned");
  TpExchangeArgs a;
  memset(&a, 0, sizeof(a));
  a.local = local;
  for (int g = 0; g < n_parts; ++g) {
    if (!peer_parts[g] || !peer_flags[g]) return fail(SLORA_ERR_NULL, "tp_allsum: null peer pointer %d", g);
    if (!aligned16(peer_parts[g])) return fail(SLORA_ERR_ALIGN, "tp_allsum: peer buffer %d is not 16-byte aligned", g);
    a.full[g] = peer_parts[g];
    a.flags[g] = peer_flags[g];
  }
  a.counter = counter;
  a.status = status;
  a.my_part = my_part;
  a.n_parts = n_parts;
  a.nproj = 1;
  a.part_width = width;
  a.T = T;
  a.full_tokens = full_tokens;
  a.seq_state = seq_state;
  a.half = half;
  a.mode = (mode & 3) | 4;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t vecs = T * (static_cast<int64_t>(width) / 8);
  const int64_t grid = vecs < 128 * 64 ? (vecs + 127) / 128 : 64;
  int rc = dtype == SLORA_F16 ? launch(tp_exchange_kernel<__half>, grid, 128, 0, flags, s, a, "tp_exchange")
                              : launch(tp_exchange_kernel<__nv_bfloat16>, grid, 128, 0, flags, s, a, "tp_exchange");
  if (rc) return rc;
  if (!(mode & 2)) return SLORA_OK;
  const int64_t sgrid = vecs < 256 * 148 ? (vecs + 255) / 256 : 148;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(sgrid), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & SLORA_FLAG_PDL) ? 1 : 0;
  cudaError_t e;
  if (dtype == SLORA_F16) {
    e = cudaLaunchKernelEx(&cfg, tp_sum_parts_kernel<__half>, static_cast<__half*>(out),
                           static_cast<const __half*>(peer_parts[my_part]), n_parts, T, full_tokens, width);
  } else {
    e = cudaLaunchKernelEx(&cfg, tp_sum_parts_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16*>(out),
                           static_cast<const __nv_bfloat16*>(peer_parts[my_part]), n_parts, T, full_tokens, width);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "tp_sum_parts: %s", cudaGetErrorString(e));
  }
  g_launches[3].fetch_add(1, std::memory_order_relaxed);
  return SLORA_OK;
}

int slora_tp_shrink_push(const void* plan, const int64_t* ids, int nproj, const int* qkvo, int part_width,
                         const void* x, int64_t x_stride, int h_in, const void* pool_a, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         int64_t n_adapters, int64_t loc_len, int64_t T, void* const* peer_full,
                         int32_t* const* peer_flags, int32_t* counter, int32_t* seq_state, int my_part, int n_parts,
                         int half, int64_t full_tokens, int inband, int dtype, unsigned flags, void* stream) {
  if (!qkvo || !peer_full || !peer_flags || !counter || !seq_state) return fail(SLORA_ERR_NULL, "null argument");
  if (n_parts < 1 || n_parts > kTpMaxParts || my_part < 0 || my_part >= n_parts || half < 0 || half > 1 ||
      full_tokens < T || part_width < 1)
    return fail(SLORA_ERR_SHAPE, "tp_shrink_push: bad part, half or buffer size");
  TpLink tp;
  memset(&tp, 0, sizeof(tp));
  for (int g = 0; g < n_parts; ++g) {
    if (!peer_full[g] || !peer_flags[g]) return fail(SLORA_ERR_NULL, "tp_shrink_push: null peer pointer %d", g);
    tp.full[g] = peer_full[g];
    tp.flags[g] = peer_flags[g];
  }
  tp.counter = counter;
  tp.seq_state = seq_state;
  tp.full_tokens = full_tokens;
  tp.my_part = my_part;
  tp.n_parts = n_parts;
  tp.half = half;
  tp.inband = (inband == 2 || inband == 3) ? inband : (inband ? 1 : 0);
  TileSrc src;
  int32_t* status;
  int rc = make_src(plan, ids, T, n_adapters, flags & SLORA_FLAG_RESOLVED_MASK, &src, &status);
  if (rc) return rc;
  if (T == 0) return SLORA_OK;  // every rank sees the same empty batch and skips the exchange
  void* d[3] = {peer_full[my_part], peer_full[my_part], peer_full[my_part]};  // unused: results go to every rank
  return run_shrink(src, make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride), pool_a, x,
                    x_stride, h_in, nproj, qkvo, d, part_width, part_width, dtype, flags, status,
                    static_cast<cudaStream_t>(stream), &tp);
}

int slora_tp_expand_wait(const void* plan, const int64_t* ids, int nproj, const int* qkvo, void* const* y,
                         const int64_t* y_stride, const int* h_out, const void* pool_b, int64_t pool_rows,
                         int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                         const void* scales, int64_t n_adapters, int64_t loc_len, int64_t T, void* my_full,
                         int32_t* my_flags, int32_t* counter, int32_t* seq_state, int my_part, int n_parts, int half,
                         int64_t full_tokens, int part_width, int inband, int dtype, unsigned flags, void* stream) {
  if (!qkvo || !y || !y_stride || !h_out || !my_full || !my_flags || !counter || !seq_state)
    return fail(SLORA_ERR_NULL, "null argument");
  if (n_parts < 1 || n_parts > kTpMaxParts || my_part < 0 || my_part >= n_parts || half < 0 || half > 1 ||
      full_tokens < T || part_width < 1 || nproj < 1 || nproj > 3)
    return fail(SLORA_ERR_SHAPE, "tp_expand_wait: bad part, half or buffer size");
  TpLink tp;
  memset(&tp, 0, sizeof(tp));
  tp.flags[my_part] = my_flags;
  tp.counter = counter;
  tp.seq_state = seq_state;
  tp.full_tokens = full_tokens;
  tp.my_part = my_part;
  tp.n_parts = n_parts;
  tp.half = half;
  tp.inband = (inband == 2 || inband == 3) ? inband : (inband ? 1 : 0);
  const int R = n_parts * part_width;
  const void* d[3];
  const int first = inband == 3 ? 0 : half;  // rotating thirds: the kernel adds the exchange's part itself
  for (int p = 0; p < 3; ++p)
    d[p] = static_cast<const char*>(my_full) + ((static_cast<int64_t>(first) * 3 + p) * full_tokens) * R * 2;
  TileSrc src;
  int32_t* status;
  int rc = make_src(plan, ids, T, n_adapters, flags & SLORA_FLAG_RESOLVED_MASK, &src, &status);
  if (rc) return rc;
  if (T == 0) return SLORA_OK;
  const Tables tb = make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride);
  rc = run_expand(src, tb, pool_b, scales, nproj, qkvo, y, y_stride, h_out, d, R, R, 1, 0, n_parts, dtype, flags,
                  status, static_cast<cudaStream_t>(stream), &tp);
  if ((rc == SLORA_ERR_ALIGN || rc == SLORA_ERR_SHAPE) && strstr(g_err, "No suitable kernel") && !inband) {
    // a layout the pipelined expand does not take: nothing has been launched yet; wait for the flags with a
    // one-CTA launch of the exchange kernel (mode 2), then expand with whatever kernel family fits
    TpExchangeArgs w;
    memset(&w, 0, sizeof(w));
    w.flags[my_part] = my_flags;
    w.counter = counter;
    w.status = status;
    w.my_part = my_part;
    w.n_parts = n_parts;
    w.nproj = 1;
    w.part_width = part_width;
    w.T = T;
    w.full_tokens = full_tokens;
    w.n_adapters = n_adapters;
    w.seq_state = seq_state;
    w.half = half;
    w.mode = 2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = dtype == SLORA_F16 ? launch(tp_exchange_kernel<__half>, 1, 128, 0, flags, s, w, "tp_exchange")
                            : launch(tp_exchange_kernel<__nv_bfloat16>, 1, 128, 0, flags, s, w, "tp_exchange");
    if (rc) return rc;
    rc = run_expand(src, tb, pool_b, scales, nproj, qkvo, y, y_stride, h_out, d, R, R, 1, 0, n_parts, dtype, flags,
                    status, s);
  }
  return rc;
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

int slora_batch_lora_qkv_rope(const void* plan, const int64_t* ids, void* q, void* k, void* v, int64_t q_stride,
                              int64_t k_stride, int64_t v_stride, int h_out_q, int h_out_kv, const void* x,
                              int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                              int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                              const void* scales, int64_t n_adapters, int64_t loc_len, void* delta_q, void* delta_k,
                              void* delta_v, int64_t delta_stride, int delta_width, int64_t T, int dtype,
                              unsigned flags, void* stream, const void* cos, const void* sin, int64_t cs_stride,
                              int head_dim, const int64_t* kv_rows, void* k_out, void* v_out, int64_t kv_out_stride,
                              int64_t kv_out_rows) {
  if (!cos || !sin) return fail(SLORA_ERR_NULL, "cos or sin is null");
  if (head_dim <= 0 || head_dim % 2 != 0 || h_out_q % head_dim != 0 || h_out_kv % head_dim != 0)
    return fail(SLORA_ERR_SHAPE, "head_dim=%d must be even and divide the q and k/v widths", head_dim);
  if ((k_out != nullptr) != (v_out != nullptr) || (k_out != nullptr && !kv_rows))
    return fail(SLORA_ERR_NULL, "k_out, v_out and kv_rows go together");
  if (k_out && (!aligned16(k_out) || !aligned16(v_out) || kv_out_stride % 8 != 0 || kv_out_rows <= 0))
    return fail(SLORA_ERR_ALIGN, "the KV destination buffers need 16-byte aligned rows");
  const int qkvo[3] = {0, 1, 2};
  void* d[3] = {delta_q, delta_k, delta_v};
  int rc = slora_lora_shrink_multi(plan, ids, 3, qkvo, d, delta_stride, delta_width, x, x_stride, h_in, pool_a,
                                   pool_rows, pool_stride, start, ranks4, loc, n_adapters, loc_len, T, dtype, flags,
                                   stream);
  if (rc) return rc;
  if (T == 0) return SLORA_OK;
  void* y[3] = {q, k, v};
  const int64_t ys[3] = {q_stride, k_stride, v_stride};
  const int ho[3] = {h_out_q, h_out_kv, h_out_kv};
  const void* dc[3] = {delta_q, delta_k, delta_v};
  RopeArgs e;
  memset(&e, 0, sizeof(e));
  e.cos = cos;
  e.sin = sin;
  e.cs_stride = cs_stride;
  e.rope_mask = 3;  // q and k
  e.out_rows = kv_rows;
  e.out[1] = k_out;
  e.out[2] = v_out;
  e.out_stride[1] = e.out_stride[2] = kv_out_stride;
  e.out_rows_limit = kv_out_rows;
  TileSrc src;
  int32_t* status;
  rc = make_src(plan, ids, T, n_adapters, flags, &src, &status);
  if (rc) return rc;
  const Tables tb = make_tables(start, ranks4, loc, n_adapters, loc_len, pool_rows, pool_stride);
  // SLORA_ROPE_EPILOGUE=0 keeps the two steps a pass of their own (A/B timing)
  static const bool epilogue_on = [] {
    const char* v = getenv("SLORA_ROPE_EPILOGUE");
    return !(v && strcmp(v, "0") == 0);
  }();
  const bool in_epilogue = epilogue_on && head_dim == kRopeHeadDim && h_out_q % kRopeHeadDim == 0 &&
                           h_out_kv % kRopeHeadDim == 0 && src.seg_split == 0 && kernel_choice() != CHOOSE_SIMPLE;
  if (in_epilogue) {
    rc = run_expand(src, tb, pool_b, scales, 3, qkvo, y, ys, ho, dc, delta_stride, delta_width, 1, 0, 1, dtype, flags,
                    status, static_cast<cudaStream_t>(stream), nullptr, &e);
    if (!(rc != SLORA_OK && strstr(g_err, "No suitable kernel"))) return rc;
  }
  // another kernel family serves this call's expand: the two steps follow as a pass of their own
  rc = run_expand(src, tb, pool_b, scales, 3, qkvo, y, ys, ho, dc, delta_stride, delta_width, 1, 0, 1, dtype, flags,
                  status, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(T), 3, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & SLORA_FLAG_PDL) ? 1 : 0;
  cudaError_t err;
  if (dtype == SLORA_F16) {
    err = cudaLaunchKernelEx(&cfg, rope_scatter_kernel<__half>, static_cast<__half*>(q), static_cast<__half*>(k),
                             static_cast<__half*>(v), q_stride, k_stride, v_stride, h_out_q, h_out_kv, h_out_kv, 3,
                             head_dim, e, status);
  } else {
    err = cudaLaunchKernelEx(&cfg, rope_scatter_kernel<__nv_bfloat16>, static_cast<__nv_bfloat16*>(q),
                             static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v), q_stride, k_stride,
                             v_stride, h_out_q, h_out_kv, h_out_kv, 3, head_dim, e, status);
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "rope_scatter: %s", cudaGetErrorString(err));
  }
  g_launches[0].fetch_add(1, std::memory_order_relaxed);
  return SLORA_OK;
}

// ---- entry point that allocates nothing ------------------------------------------------------------------------
// Scratch of slora_batch_lora_o_noalloc: the batch plan (first kNoAllocPlanBytes) and the rank-r intermediate of up to
// kNoAllocMaxTokens tokens x 128 columns.  One copy per GPU that loads the library, held until the process exits and
// shared by every call on that GPU.
constexpr int64_t kNoAllocMaxTokens = 1024;
constexpr int64_t kNoAllocMaxAdapters = 4096;
constexpr size_t kNoAllocPlanBytes = 64 * 1024;
constexpr size_t kNoAllocDeltaBytes = static_cast<size_t>(kNoAllocMaxTokens) * 128 * 2;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPlanBytes + kNoAllocDeltaBytes];

// Device address of the scratch array on the current device.  In host code the array's name is only a handle; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.  The
// per-device cache is a set of atomics: two host threads that make the first call on a device at the same time both
// look the address up and store the same value.
static int noalloc_scratch(unsigned char** out) {
  static std::atomic<unsigned char*> addr[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(SLORA_ERR_LAUNCH, "cudaGetDevice: %s", e == cudaSuccess ? "device index out of range" : cudaGetErrorString(e));
  }
  unsigned char* known = addr[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(SLORA_ERR_LAUNCH, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
    }
    known = static_cast<unsigned char*>(p);
    addr[dev].store(known, std::memory_order_release);
  }
  *out = known;
  return SLORA_OK;
}

int slora_batch_lora_o_noalloc(const int64_t* ids, void* o, int64_t o_stride, int h_out, const void* x,
                               int64_t x_stride, int h_in, const void* pool_a, const void* pool_b, int64_t pool_rows,
                               int64_t pool_stride, const int64_t* start, const int64_t* ranks4, const int64_t* loc,
                               const void* scales, int64_t n_adapters, int64_t loc_len, int max_rank, int64_t T,
                               int dtype, unsigned flags, void* stream) {
  if (T < 0 || T > kNoAllocMaxTokens)
    return fail(SLORA_ERR_WORKSPACE, "slora_batch_lora_o_noalloc: T=%lld exceeds the built-in scratch (max %lld tokens)",
                (long long)T, (long long)kNoAllocMaxTokens);
  if (n_adapters < 0 || n_adapters > kNoAllocMaxAdapters)
    return fail(SLORA_ERR_WORKSPACE, "slora_batch_lora_o_noalloc: n_adapters=%lld exceeds the built-in scratch (max %lld)",
                (long long)n_adapters, (long long)kNoAllocMaxAdapters);
  if (max_rank <= 0 || max_rank > 128 || max_rank % 8 != 0)
    return fail(SLORA_ERR_RANK, "slora_batch_lora_o_noalloc: max_rank=%d must be a multiple of 8 up to 128", max_rank);
  if (slora_plan_workspace_bytes(T, n_adapters) > kNoAllocPlanBytes)
    return fail(SLORA_ERR_WORKSPACE, "slora_batch_lora_o_noalloc: plan of %zu bytes exceeds the built-in %zu",
                slora_plan_workspace_bytes(T, n_adapters), kNoAllocPlanBytes);
  unsigned char* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  if (T == 0) return SLORA_OK;
  // Routing big same-adapter groups to the tensor-core kernels may fork to a library-owned side stream, which is
  // created (stream and events) at first use: not in a call that promises to allocate nothing.  The bit is dropped;
  // such groups run on the CUDA-core kernels here.
  flags &= ~static_cast<unsigned>(SLORA_FLAG_BIG_GROUPS | SLORA_FLAG_RESOLVED_MASK);  // its plan has no resolved tiles
  // the plan kernel clears its own counters; the intermediate needs no clearing (only columns < r are written and read)
  rc = slora_plan_build(scratch, kNoAllocPlanBytes, ids, T, start, ranks4, n_adapters, loc_len, stream);
  if (rc) return rc;
  return slora_batch_lora_o(scratch, ids, o, o_stride, h_out, x, x_stride, h_in, pool_a, pool_b, pool_rows, pool_stride,
                            start, ranks4, loc, scales, n_adapters, loc_len, scratch + kNoAllocPlanBytes, max_rank,
                            max_rank, T, dtype, flags, stream);
}

int slora_noalloc_status(int* status_out, void* stream) {
  if (!status_out) return fail(SLORA_ERR_NULL, "status_out is null");
  unsigned char* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  int32_t hdr[PH_WORDS];
  cudaError_t e = cudaMemcpyAsync(hdr, scratch, sizeof(hdr), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(SLORA_ERR_LAUNCH, "noalloc_status: %s", cudaGetErrorString(e));
  // before the first call on this device the scratch holds no plan: nothing to report
  *status_out = hdr[PH_MAGIC] == kPlanMagic ? hdr[PH_STATUS] : 0;
  return SLORA_OK;
}

int slora_tp_regroup(void* out, const void* gathered, const int64_t* ids, const int64_t* ranks4, int n_parts,
                     int nproj, int64_t T, int part_width, int64_t part_stride, int64_t n_adapters, int dtype,
                     void* stream) {
  if (T == 0) return SLORA_OK;
  if (!out || !gathered || !ids || !ranks4) return fail(SLORA_ERR_NULL, "null buffer or table pointer");
  if (dtype != SLORA_F16 && dtype != SLORA_BF16) return fail(SLORA_ERR_DTYPE, "unsupported dtype %d", dtype);
  if (n_parts < 1 || nproj < 1 || nproj > 3 || part_width < 1 || T < 0 || T > 0x7fffffff || part_stride < 0)
    return fail(SLORA_ERR_SHAPE, "tp_regroup: bad shape");
  const dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>(nproj));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == SLORA_F16) {
    tp_regroup_kernel<__half><<<grid, 128, 0, s>>>(static_cast<__half*>(out), static_cast<const __half*>(gathered), ids,
                                                  ranks4, n_parts, part_width, T, part_stride, n_adapters);
  } else {
    tp_regroup_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(static_cast<__nv_bfloat16*>(out),
                                                         static_cast<const __nv_bfloat16*>(gathered), ids, ranks4,
                                                         n_parts, part_width, T, part_stride, n_adapters);
  }
  return check_launch("tp_regroup", 1);
}

int slora_tp_exchange(const void* local, void* const* peer_full, int32_t* const* peer_flags, int32_t* counter,
                      int32_t* status, const int64_t* ids, const int64_t* ranks4, int my_part, int n_parts, int nproj,
                      int64_t T, int64_t full_tokens, int part_width, int64_t n_adapters, int half, int32_t* seq_state,
                      int mode, int dtype, unsigned flags, void* stream) {
  if (full_tokens < T) return fail(SLORA_ERR_SHAPE, "tp_exchange: delta buffers hold %lld token rows, batch has %lld",
                                   (long long)full_tokens, (long long)T);
  if (dtype != SLORA_F16 && dtype != SLORA_BF16) return fail(SLORA_ERR_DTYPE, "unsupported dtype %d", dtype);
  if (!peer_full || !peer_flags || !counter || !seq_state) return fail(SLORA_ERR_NULL, "null peer table or counter");
  if (n_parts < 1 || n_parts > kTpMaxParts || my_part < 0 || my_part >= n_parts)
    return fail(SLORA_ERR_SHAPE, "tp_exchange: n_parts=%d (max %d), my_part=%d", n_parts, kTpMaxParts, my_part);
  if (nproj < 1 || nproj > 3 || part_width < 1 || T < 0 || T > 0x7fffffff || half < 0 || half > 1 || (mode & 3) == 0)
    return fail(SLORA_ERR_SHAPE, "tp_exchange: bad shape, half or mode");
  if ((mode & 1) && T > 0 && (!local || !ids || !ranks4)) return fail(SLORA_ERR_NULL, "null buffer or table pointer");
  TpExchangeArgs a;
  memset(&a, 0, sizeof(a));
  a.local = local;
  for (int g = 0; g < n_parts; ++g) {
    if (!peer_full[g] || !peer_flags[g]) return fail(SLORA_ERR_NULL, "tp_exchange: null peer pointer %d", g);
    a.full[g] = peer_full[g];
    a.flags[g] = peer_flags[g];
  }
  a.counter = counter;
  a.status = status;
  a.ids = ids;
  a.ranks4 = ranks4;
  a.my_part = my_part;
  a.n_parts = n_parts;
  a.nproj = nproj;
  a.part_width = part_width;
  a.T = T;
  a.full_tokens = full_tokens;
  a.n_adapters = n_adapters;
  a.seq_state = seq_state;
  a.half = half;
  a.mode = mode;
  const bool push = (mode & 1) && T > 0;
  const int64_t grid = push ? (T + kTpTokensPerCta - 1) / kTpTokensPerCta * nproj : 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  if (dtype == SLORA_F16) {
    rc = launch(tp_exchange_kernel<__half>, grid, 128, 0, flags, s, a, "tp_exchange");
  } else {
    rc = launch(tp_exchange_kernel<__nv_bfloat16>, grid, 128, 0, flags, s, a, "tp_exchange");
  }
  return rc;
}

int slora_pool_scatter_rows(void* const* key_buffers, void* const* value_buffers, const void* const* src, int n_layers,
                            const int64_t* loc, int64_t n_rows, int64_t row_bytes, int64_t pool_rows,
                            int64_t pool_row_bytes, int32_t* status, void* stream) {
  if (n_rows == 0 || n_layers == 0) return SLORA_OK;
  if (!key_buffers || !value_buffers || !src || !loc) return fail(SLORA_ERR_NULL, "null pointer table or loc");
  if (n_layers < 0 || n_rows < 0 || n_rows > 0x7fffffff || pool_rows <= 0)
    return fail(SLORA_ERR_SHAPE, "pool_scatter_rows: bad sizes");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || pool_row_bytes < row_bytes || pool_row_bytes % 16 != 0)
    return fail(SLORA_ERR_ALIGN, "pool_scatter_rows: rows must be multiples of 16 bytes and fit a pool row");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int l0 = 0; l0 < n_layers; l0 += kScatterLayers) {
    PoolScatterArgs a;
    memset(&a, 0, sizeof(a));
    a.n_layers = n_layers - l0 < kScatterLayers ? n_layers - l0 : kScatterLayers;
    for (int l = 0; l < a.n_layers; ++l) {
      if (!key_buffers[l0 + l] || !value_buffers[l0 + l] || !src[l0 + l])
        return fail(SLORA_ERR_NULL, "pool_scatter_rows: null buffer of layer %d", l0 + l);
      if (!aligned16(key_buffers[l0 + l]) || !aligned16(value_buffers[l0 + l]) || !aligned16(src[l0 + l]))
        return fail(SLORA_ERR_ALIGN, "pool_scatter_rows: buffer of layer %d is not 16-byte aligned", l0 + l);
      a.key[l] = key_buffers[l0 + l];
      a.value[l] = value_buffers[l0 + l];
      a.src[l] = src[l0 + l];
    }
    a.loc = loc;
    a.n_rows = n_rows;
    a.row_bytes = row_bytes;
    a.pool_rows = pool_rows;
    a.pool_row_bytes = pool_row_bytes;
    a.status = status;
    const dim3 grid(static_cast<unsigned>(n_rows), 2, static_cast<unsigned>(a.n_layers));
    pool_scatter_kernel<<<grid, 256, 0, s>>>(a);
    const int rc = check_launch("pool_scatter_rows", 1);
    if (rc) return rc;
  }
  return SLORA_OK;
}

size_t slora_pool_alloc_workspace_bytes(int64_t tot_rows) {
  if (tot_rows <= 0) return 0;
  return static_cast<size_t>((tot_rows + kPoolSegRows - 1) / kPoolSegRows) * sizeof(int32_t);
}

int slora_pool_alloc_rows(uint8_t* mem_state, int64_t tot_rows, int64_t need, int64_t* out_rows, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream) {
  if (need == 0) return SLORA_OK;
  if (!mem_state || !out_rows || !workspace) return fail(SLORA_ERR_NULL, "pool_alloc_rows: null free map, output or workspace");
  if (tot_rows <= 0 || need < 0 || need > tot_rows) return fail(SLORA_ERR_SHAPE, "pool_alloc_rows: bad sizes");
  if (!aligned16(mem_state)) return fail(SLORA_ERR_ALIGN, "pool_alloc_rows: the free map must be 16-byte aligned");
  if (workspace_bytes < slora_pool_alloc_workspace_bytes(tot_rows))
    return fail(SLORA_ERR_WORKSPACE, "pool_alloc_rows: workspace of %zu bytes, %zu needed", workspace_bytes,
                slora_pool_alloc_workspace_bytes(tot_rows));
  const int64_t segs = (tot_rows + kPoolSegRows - 1) / kPoolSegRows;
  if (segs > 0x7fffffff) return fail(SLORA_ERR_SHAPE, "pool_alloc_rows: free map too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* seg_free = static_cast<int32_t*>(workspace);
  pool_count_kernel<<<static_cast<unsigned>(segs), kPoolThreads, 0, s>>>(mem_state, tot_rows, seg_free);
  pool_take_kernel<<<static_cast<unsigned>(segs), kPoolThreads, 0, s>>>(mem_state, tot_rows, seg_free, need, out_rows,
                                                                        status);
  return check_launch("pool_alloc_rows", 2);
}

int slora_pool_free_rows(uint8_t* mem_state, int64_t tot_rows, const int64_t* rows, int64_t n, int32_t* status,
                         void* stream) {
  if (n == 0) return SLORA_OK;
  if (!mem_state || !rows) return fail(SLORA_ERR_NULL, "pool_free_rows: null free map or row list");
  if (tot_rows <= 0 || n < 0) return fail(SLORA_ERR_SHAPE, "pool_free_rows: bad sizes");
  const int64_t blocks = (n + 255) / 256;
  pool_free_kernel<<<static_cast<unsigned>(blocks < 1184 ? blocks : 1184), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mem_state, tot_rows, rows, n, status);
  return check_launch("pool_free_rows", 1);
}

int slora_tables_compact(const int64_t* a_start, const int64_t* a_len, const int64_t* a_loc, const void* a_scaling,
                         const uint8_t* keep, int64_t n_adapters, int64_t loc_len, int64_t* new_start,
                         int64_t* new_len, int64_t* new_loc, void* new_scaling, int64_t* scratch, int64_t* counts,
                         uint8_t* mem_state, int64_t tot_rows, int32_t* status, void* stream) {
  if (n_adapters == 0) return SLORA_OK;
  if (!a_start || !a_len || !a_loc || !a_scaling || !keep || !new_start || !new_len || !new_loc || !new_scaling ||
      !scratch)
    return fail(SLORA_ERR_NULL, "tables_compact: null table, output or scratch");
  if (n_adapters < 0 || loc_len < 0 || (mem_state != nullptr && tot_rows <= 0))
    return fail(SLORA_ERR_SHAPE, "tables_compact: bad sizes");
  if (new_loc == a_loc || new_start == a_start || new_len == a_len || new_scaling == a_scaling)
    return fail(SLORA_ERR_SHAPE, "tables_compact: the new tables must not be the old ones");
  CompactArgs a;
  a.a_start = a_start;
  a.a_len = a_len;
  a.a_loc = a_loc;
  a.a_scaling = static_cast<const uint16_t*>(a_scaling);
  a.keep = keep;
  a.n_adapters = n_adapters;
  a.loc_len = loc_len;
  a.new_start = new_start;
  a.new_len = new_len;
  a.new_loc = new_loc;
  a.new_scaling = static_cast<uint16_t*>(new_scaling);
  a.dst_off = scratch;
  a.counts = counts;
  a.mem_state = mem_state;
  a.tot = tot_rows;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  tables_scan_kernel<<<1, kPoolThreads, 0, s>>>(a);
  tables_move_kernel<<<static_cast<unsigned>((n_adapters + 7) / 8), 256, 0, s>>>(a);
  return check_launch("tables_compact", 2);
}

int slora_validate_tables(const int64_t* start, const int64_t* ranks4, const int64_t* loc, const int64_t* ids,
                          int64_t n_adapters, int64_t loc_len, int64_t T, int64_t pool_rows, int32_t* report,
                          void* stream) {
  if (!start || !ranks4 || !loc || !report) return fail(SLORA_ERR_NULL, "null table or report pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  zero_report_kernel<<<1, 32, 0, s>>>(report);
  validate_tables_kernel<<<64, 256, 0, s>>>(start, ranks4, loc, ids, n_adapters, loc_len, T, pool_rows, report);
  return check_launch("validate_tables", 2);
}

}  // extern "C"
