// Unified-Paging pool bookkeeping on the device: row allocation from the free map and compaction of the adapter
// tables when adapters are dropped.  Integer and byte work only; every kernel is bounded by the size of its tables.
//
// What the reference does for the same steps:
//   alloc   slora/common/mem_allocator.py:30-39    cumulative sum over the whole free map, mask, nonzero -> the first
//                                                  `need` free rows in increasing order, marked used
//   free    slora/common/mem_allocator.py:185-199  mem_state[rows] = 1
//   offload slora/server/router/model_infer/infer_adapter.py:186-250  kept adapters keep their order; a_len / a_scaling
//                                                  gathered, a_start = exclusive prefix sum of the kept lengths,
//                                                  a_loc runs copied by a variable-length copy kernel, rows of the
//                                                  dropped adapters freed
#pragma once
#include <cstdint>

#include "lora_common.cuh"

namespace slora {

constexpr int kPoolThreads = 1024;
constexpr int kPoolBytesPerThread = 16;
constexpr int64_t kPoolSegRows = static_cast<int64_t>(kPoolThreads) * kPoolBytesPerThread;  // free-map rows per CTA

// Inclusive scan of one int per thread over a 1024-thread CTA; returns the thread's inclusive value, *total = sum.
__device__ __forceinline__ int block_scan_inclusive(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += n;
  }
  if (lane == 31) warp_sums[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += n;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int before = warp == 0 ? 0 : warp_sums[warp - 1];
  *total = warp_sums[31];
  __syncthreads();  // warp_sums may be reused by the caller
  return v + before;
}

// The 16 free-map bytes of this thread (zero beyond the end of the map); the map is 16-byte aligned.
__device__ __forceinline__ uint4 pool_load16(const uint8_t* mem_state, int64_t pos, int64_t tot) {
  uint4 v = make_uint4(0, 0, 0, 0);
  if (pos + kPoolBytesPerThread <= tot) {
    v = *reinterpret_cast<const uint4*>(mem_state + pos);
  } else if (pos < tot) {
    uint8_t* b = reinterpret_cast<uint8_t*>(&v);
    for (int i = 0; i < tot - pos; ++i) b[i] = mem_state[pos + i];
  }
  return v;
}
__device__ __forceinline__ int pool_count16(const uint4& v) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
  int c = 0;
#pragma unroll
  for (int i = 0; i < kPoolBytesPerThread; ++i) c += b[i] != 0;
  return c;
}

// Pass 1 of the allocation: free rows in each segment of kPoolSegRows rows.
__global__ void __launch_bounds__(kPoolThreads) pool_count_kernel(const uint8_t* __restrict__ mem_state, int64_t tot,
                                                                  int32_t* __restrict__ seg_free) {
  __shared__ int warp_sums[32];
  const int64_t pos = blockIdx.x * kPoolSegRows + static_cast<int64_t>(threadIdx.x) * kPoolBytesPerThread;
  int total;
  block_scan_inclusive(pool_count16(pool_load16(mem_state, pos, tot)), warp_sums, &total);
  if (threadIdx.x == 0) seg_free[blockIdx.x] = total;
}

// Pass 2: segment s hands out the free rows whose ordinal (count of free rows before them in the whole map) is below
// `need`, writes them to out_rows[ordinal] and marks them used.  The last segment also reports a shortfall: fewer
// free rows in the map than asked for (the caller's own count was wrong) -> the missing entries become -1.
__global__ void __launch_bounds__(kPoolThreads) pool_take_kernel(uint8_t* __restrict__ mem_state, int64_t tot,
                                                                 const int32_t* __restrict__ seg_free, int64_t need,
                                                                 int64_t* __restrict__ out_rows,
                                                                 int32_t* __restrict__ status) {
  __shared__ int warp_sums[32];
  __shared__ long long s_before;
  const int seg = blockIdx.x, tid = threadIdx.x;
  // free rows before this segment: sum of the earlier segments' counts
  long long part = 0;
  for (int i = tid; i < seg; i += kPoolThreads) part += seg_free[i];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) part += __shfl_down_sync(0xffffffffu, part, d);
  if (tid == 0) s_before = 0;
  __syncthreads();
  if ((tid & 31) == 0 && part != 0) atomicAdd(reinterpret_cast<unsigned long long*>(&s_before), static_cast<unsigned long long>(part));
  __syncthreads();
  const long long before = s_before;
  if (seg == static_cast<int>(gridDim.x) - 1) {
    const long long have = before + seg_free[seg];
    if (have < need) {
      if (tid == 0) set_status(status, SLORA_STATUS_BAD_TABLE);
      for (long long i = have + tid; i < need; i += kPoolThreads) out_rows[i] = -1;
    }
  }
  if (before >= need) return;  // uniform over the CTA
  const int64_t pos = seg * kPoolSegRows + static_cast<int64_t>(tid) * kPoolBytesPerThread;
  uint4 v = pool_load16(mem_state, pos, tot);
  const int mine = pool_count16(v);
  int total;
  const int incl = block_scan_inclusive(mine, warp_sums, &total);
  long long ord = before + incl - mine;
  if (mine == 0 || ord >= need) return;
  uint8_t* b = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
  for (int i = 0; i < kPoolBytesPerThread; ++i) {
    if (b[i] != 0 && ord < need) {
      out_rows[ord++] = pos + i;
      b[i] = 0;
    }
  }
  if (pos + kPoolBytesPerThread <= tot) {
    *reinterpret_cast<uint4*>(mem_state + pos) = v;
  } else {
    for (int i = 0; i < tot - pos; ++i) mem_state[pos + i] = b[i];
  }
}

__global__ void __launch_bounds__(256) pool_free_kernel(uint8_t* __restrict__ mem_state, int64_t tot,
                                                        const int64_t* __restrict__ rows, int64_t n,
                                                        int32_t* __restrict__ status) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = rows[i];
    if (r < 0 || r >= tot) {
      set_status(status, SLORA_STATUS_BAD_TABLE);
      continue;
    }
    mem_state[r] = 1;
  }
}

struct CompactArgs {
  const int64_t* a_start;
  const int64_t* a_len;
  const int64_t* a_loc;
  const uint16_t* a_scaling;  // 2-byte elements (fp16 / bf16), copied as bits
  const uint8_t* keep;        // one byte per adapter, non-zero = stays resident
  int64_t n_adapters, loc_len;
  int64_t* new_start;
  int64_t* new_len;
  int64_t* new_loc;
  uint16_t* new_scaling;
  int64_t* dst_off;  // scratch, one per adapter: where its run goes in new_loc, -1 = dropped
  int64_t* counts;   // [0] adapters kept, [1] rows kept (may be null)
  uint8_t* mem_state;
  int64_t tot;
  int32_t* status;
};

// Pass 1 of the compaction, one CTA: position of every kept adapter in the new tables (exclusive scans of the keep
// flags and of the kept lengths, in the adapters' order).
__global__ void __launch_bounds__(kPoolThreads) tables_scan_kernel(const CompactArgs a) {
  __shared__ int warp_sums[32];
  long long kept = 0, rows = 0;
  for (int64_t base = 0; base < a.n_adapters; base += kPoolThreads) {
    const int64_t i = base + threadIdx.x;
    const bool in = i < a.n_adapters;
    bool ok = false;
    int k = 0, len = 0;
    if (in) {
      const int64_t l = a.a_len[i], s = a.a_start[i];
      ok = l >= 0 && s >= 0 && s + l <= a.loc_len && l <= 0x7fffffff;
      if (!ok) set_status(a.status, SLORA_STATUS_BAD_TABLE);
      k = ok && a.keep[i] != 0;
      len = k ? static_cast<int>(l) : 0;
    }
    int tk, tl;
    const int ik = block_scan_inclusive(k, warp_sums, &tk);
    const int il = block_scan_inclusive(len, warp_sums, &tl);
    if (in) {
      if (!ok) {
        a.dst_off[i] = -2;  // a broken entry is neither copied nor freed
      } else if (k) {
        const long long slot = kept + ik - 1, off = rows + il - len;
        a.new_start[slot] = off;
        a.new_len[slot] = len;
        a.new_scaling[slot] = a.a_scaling[i];
        a.dst_off[i] = off;
      } else {
        a.dst_off[i] = -1;
      }
    }
    kept += tk;
    rows += tl;
  }
  if (threadIdx.x == 0 && a.counts != nullptr) {
    a.counts[0] = kept;
    a.counts[1] = rows;
  }
}

// Pass 2, one warp per adapter: a kept adapter's run of a_loc moves to its new place, a dropped adapter's rows go
// back to the free map.
__global__ void __launch_bounds__(256) tables_move_kernel(const CompactArgs a) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= a.n_adapters) return;
  const int lane = threadIdx.x & 31;
  const int64_t off = a.dst_off[i];
  if (off == -2) return;
  const int64_t s = a.a_start[i], l = a.a_len[i];
  if (off >= 0) {
    for (int64_t j = lane; j < l; j += 32) a.new_loc[off + j] = a.a_loc[s + j];
  } else if (a.mem_state != nullptr) {
    for (int64_t j = lane; j < l; j += 32) {
      const int64_t r = a.a_loc[s + j];
      if (r < 0 || r >= a.tot) {
        set_status(a.status, SLORA_STATUS_BAD_TABLE);
        continue;
      }
      a.mem_state[r] = 1;
    }
  }
}

}  // namespace slora
