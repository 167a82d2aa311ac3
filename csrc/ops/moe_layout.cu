// Expert-grouped row layout of a routed batch, built on the device without a sort and without a host round trip.
//
// Input: the expert of every routed entry (token x slot). Output: a stable counting sort of the entries of THIS rank's
// experts into rows, each expert's range padded to whole 128-row tiles:
//   dest_row[entry]   row of the entry (-1: another rank's expert, or dropped because the row buffer is full)
//   src_entry[row]    entry held by the row (-1: padding)
//   tile_expert[tile] local expert of each 128-row tile (num_local for unused tiles)
//   padded_offsets    first row of every expert (+ end)
//   dropped           number of entries that did not fit into `rows` (0 unless a capacity bound is in force)
// Three launches: per-chunk histograms, one block that turns them into offsets, and the stable placement (inside a
// chunk every warp ranks its entries with match/ballot, so equal experts keep their order and the result is
// reproducible bit for bit).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "../common/launch.h"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPerWarp = 256;                 // entries per warp: 8 steps of 32
constexpr int kChunk = kWarps * kPerWarp;     // entries per block
constexpr int kMaxLocal = 256;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

__device__ __forceinline__ int local_expert(int e, int first, int num_local) {
  const int l = e - first;
  return (l >= 0 && l < num_local) ? l : -1;
}

// counts[block][expert] = entries of the block's chunk that go to the local expert
__global__ void layout_count_kernel(const int* __restrict__ expert_of_entry, int entries, int first, int num_local,
                                    int* __restrict__ counts) {
  __shared__ int hist[kMaxLocal];
  for (int i = threadIdx.x; i < num_local; i += kThreads) hist[i] = 0;
  __syncthreads();
  const int base = blockIdx.x * kChunk;
  for (int i = threadIdx.x; i < kChunk; i += kThreads) {
    const int idx = base + i;
    if (idx < entries) {
      const int l = local_expert(expert_of_entry[idx], first, num_local);
      if (l >= 0) atomicAdd(&hist[l], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < num_local; i += kThreads) counts[(size_t)blockIdx.x * num_local + i] = hist[i];
}

// counts[block][expert] -> first row of that (block, expert) pair; padded_offsets; tile_expert. One block.
__global__ void layout_scan_kernel(int* __restrict__ counts, int blocks, int num_local, int rows, int* __restrict__ padded_offsets,
                                   int* __restrict__ tile_expert) {
  __shared__ int total[kMaxLocal];
  __shared__ int start[kMaxLocal + 1];
  for (int e = threadIdx.x; e < num_local; e += kThreads) {
    int run = 0;
    for (int b = 0; b < blocks; ++b) {
      const int c = counts[(size_t)b * num_local + e];
      counts[(size_t)b * num_local + e] = run;
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < num_local; ++e) {
      start[e] = min(at, rows);  // under a capacity bound the ranges past the end of the buffer are empty
      at += (total[e] + kTile - 1) / kTile * kTile;
    }
    start[num_local] = min(at, rows);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= num_local; e += kThreads) padded_offsets[e] = start[e];
  for (int e = threadIdx.x; e < num_local; e += kThreads) {
    for (int b = 0; b < blocks; ++b) counts[(size_t)b * num_local + e] += start[e];
  }
  for (int t = threadIdx.x; t < rows / kTile; t += kThreads) {
    const int row = t * kTile;
    int lo = 0, hi = num_local;  // first expert whose end is beyond `row`
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (start[mid + 1] > row) hi = mid; else lo = mid + 1;
    }
    tile_expert[t] = lo;
  }
}

// stable placement: entry -> row (block base + entries of the same expert earlier in the chunk)
__global__ void layout_place_kernel(const int* __restrict__ expert_of_entry, int entries, int first, int num_local,
                                    const int* __restrict__ base_rows, int rows, int* __restrict__ dest_row, int* __restrict__ src_entry,
                                    int* __restrict__ dropped) {
  __shared__ int wcount[kWarps][kMaxLocal];  // entries per (warp, expert), then running offsets
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kWarps * kMaxLocal; i += kThreads) (&wcount[0][0])[i] = 0;
  __syncthreads();
  const int warp_base = blockIdx.x * kChunk + warp * kPerWarp;
  int key[kPerWarp / 32];
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int idx = warp_base + s * 32 + lane;
    key[s] = idx < entries ? local_expert(expert_of_entry[idx], first, num_local) : -1;
    if (key[s] >= 0) atomicAdd(&wcount[warp][key[s]], 1);
  }
  __syncthreads();
  // exclusive prefix over the warps of the block, per expert, offset by the block's first row
  for (int e = threadIdx.x; e < num_local; e += kThreads) {
    int run = base_rows[(size_t)blockIdx.x * num_local + e];
    for (int w = 0; w < kWarps; ++w) {
      const int c = wcount[w][e];
      wcount[w][e] = run;
      run += c;
    }
  }
  __syncthreads();
  int lost = 0;
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int idx = warp_base + s * 32 + lane;
    const int k = key[s];
    // lanes with the same expert form a group; ranks inside the group follow the lane (= entry) order
    const unsigned peers = __match_any_sync(0xffffffffu, k);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int row = -1;
    if (k >= 0) {
      row = wcount[warp][k] + rank;
      if (row >= rows) {
        row = -1;
        ++lost;
      }
    }
    __syncwarp();
    if (k >= 0 && rank == 0) wcount[warp][k] += __popc(peers);
    __syncwarp();
    if (idx < entries) {
      dest_row[idx] = row;
      if (row >= 0) src_entry[row] = idx;
    }
  }
  if (lost > 0) atomicAdd(dropped, lost);
}

// -> (dest_row [entries], src_entry [rows], tile_expert [rows / 128], padded_offsets [num_local + 1], dropped [1])
std::vector<Tensor> moe_layout(const Tensor& expert_of_entry, int64_t first_expert, int64_t num_local, int64_t rows) {
  TORCH_CHECK(expert_of_entry.is_cuda() && expert_of_entry.scalar_type() == torch::kInt32 && expert_of_entry.is_contiguous(), "expert_of_entry: int32");
  TORCH_CHECK(num_local >= 1 && num_local <= kMaxLocal, "between 1 and 256 local experts");
  TORCH_CHECK(rows > 0 && rows % kTile == 0, "rows must be a positive multiple of 128");
  const c10::cuda::CUDAGuard guard(expert_of_entry.device());
  const int64_t entries = expert_of_entry.numel();
  auto opts = expert_of_entry.options();
  Tensor dest_row = torch::empty({entries}, opts);
  Tensor src_entry = torch::empty({rows}, opts);
  Tensor tile_expert = torch::empty({rows / kTile}, opts);
  Tensor padded_offsets = torch::empty({num_local + 1}, opts);
  Tensor dropped = torch::zeros({1}, opts);
  const int blocks = (int)std::max<int64_t>(1, (entries + kChunk - 1) / kChunk);
  Tensor counts = torch::empty({blocks, num_local}, opts);
  cudaStream_t stream = cur_stream();
  check_cuda(cudaMemsetAsync(src_entry.data_ptr(), 0xFF, (size_t)rows * sizeof(int), stream), "src_entry memset");
  layout_count_kernel<<<blocks, kThreads, 0, stream>>>(expert_of_entry.data_ptr<int>(), (int)entries, (int)first_expert, (int)num_local,
                                                       counts.data_ptr<int>());
  layout_scan_kernel<<<1, kThreads, 0, stream>>>(counts.data_ptr<int>(), blocks, (int)num_local, (int)rows, padded_offsets.data_ptr<int>(),
                                                 tile_expert.data_ptr<int>());
  layout_place_kernel<<<blocks, kThreads, 0, stream>>>(expert_of_entry.data_ptr<int>(), (int)entries, (int)first_expert, (int)num_local,
                                                       counts.data_ptr<int>(), (int)rows, dest_row.data_ptr<int>(),
                                                       src_entry.data_ptr<int>(), dropped.data_ptr<int>());
  count_launch(3);
  check_cuda(cudaGetLastError(), "moe_layout launch");
  return {dest_row, src_entry, tile_expert, padded_offsets, dropped};
}


// ---- the same layout for a whole expert-parallel group -------------------------------------------------------------------
// Every rank of an expert-parallel group holds the routing table of the whole group, so it can work out where EVERY entry
// lands on its owner (the rank whose experts include the entry's expert) without asking: one counting sort over all
// experts whose row offsets restart at each owner's first expert. That gives this rank its own layout (as above) and, for
// the combine, the (owner, row) of every entry, which used to take an all-to-all per layer.

// counts[block][expert] -> first row of that (block, expert) pair on the expert's owner; this rank's padded_offsets and
// tile_expert. One block.
__global__ void layout_scan_group_kernel(int* __restrict__ counts, int blocks, int num_experts, int per_owner, int my_owner, int rows,
                                         int* __restrict__ padded_offsets, int* __restrict__ tile_expert) {
  __shared__ int total[kMaxLocal];
  __shared__ int start[kMaxLocal + 1];  // start[e]: first row of expert e on its owner
  __shared__ int mine[kMaxLocal + 1];   // this rank's experts: first rows, then the end of the last one
  for (int e = threadIdx.x; e < num_experts; e += kThreads) {
    int run = 0;
    for (int b = 0; b < blocks; ++b) {
      const int c = counts[(size_t)b * num_experts + e];
      counts[(size_t)b * num_experts + e] = run;
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < num_experts; ++e) {
      if (e % per_owner == 0) at = 0;
      start[e] = min(at, rows);  // under a capacity bound the ranges past the end of the buffer are empty
      at += (total[e] + kTile - 1) / kTile * kTile;
      if (e / per_owner == my_owner) {
        mine[e % per_owner] = start[e];
        mine[e % per_owner + 1] = min(at, rows);
      }
    }
  }
  __syncthreads();
  for (int l = threadIdx.x; l <= per_owner; l += kThreads) padded_offsets[l] = mine[l];
  for (int e = threadIdx.x; e < num_experts; e += kThreads) {
    for (int b = 0; b < blocks; ++b) counts[(size_t)b * num_experts + e] += start[e];
  }
  for (int t = threadIdx.x; t < rows / kTile; t += kThreads) {
    const int row = t * kTile;
    int lo = 0, hi = per_owner;  // first local expert whose end is beyond `row`
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (mine[mid + 1] > row) hi = mid; else lo = mid + 1;
    }
    tile_expert[t] = lo;
  }
}

// stable placement over all experts: dest_row / src_entry for this rank's experts, owner * rows + row for every entry
__global__ void layout_place_group_kernel(const int* __restrict__ expert_of_entry, int entries, int num_experts, int per_owner, int my_owner,
                                          const int* __restrict__ base_rows, int rows, int* __restrict__ dest_row, int* __restrict__ src_entry,
                                          int* __restrict__ global_row, int* __restrict__ dropped) {
  __shared__ int wcount[kWarps][kMaxLocal];  // entries per (warp, expert), then running offsets
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kWarps * kMaxLocal; i += kThreads) (&wcount[0][0])[i] = 0;
  __syncthreads();
  const int warp_base = blockIdx.x * kChunk + warp * kPerWarp;
  int key[kPerWarp / 32];
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int idx = warp_base + s * 32 + lane;
    key[s] = idx < entries ? local_expert(expert_of_entry[idx], 0, num_experts) : -1;
    if (key[s] >= 0) atomicAdd(&wcount[warp][key[s]], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += kThreads) {
    int run = base_rows[(size_t)blockIdx.x * num_experts + e];
    for (int w = 0; w < kWarps; ++w) {
      const int c = wcount[w][e];
      wcount[w][e] = run;
      run += c;
    }
  }
  __syncthreads();
  int lost = 0;
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int idx = warp_base + s * 32 + lane;
    const int k = key[s];
    const unsigned peers = __match_any_sync(0xffffffffu, k);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int owner = k >= 0 ? k / per_owner : -1;
    int row = -1;
    if (k >= 0) {
      row = wcount[warp][k] + rank;
      if (row >= rows) {
        row = -1;
        if (owner == my_owner) ++lost;
      }
    }
    __syncwarp();
    if (k >= 0 && rank == 0) wcount[warp][k] += __popc(peers);
    __syncwarp();
    if (idx < entries) {
      const bool here = owner == my_owner && row >= 0;
      dest_row[idx] = here ? row : -1;
      if (here) src_entry[row] = idx;
      global_row[idx] = row >= 0 ? owner * rows + row : -1;
    }
  }
  if (lost > 0) atomicAdd(dropped, lost);
}

// -> (dest_row [entries], src_entry [rows], tile_expert [rows / 128], padded_offsets [per_owner + 1], dropped [1], global_row [entries])
std::vector<Tensor> moe_layout_group(const Tensor& expert_of_entry, int64_t num_experts, int64_t per_owner, int64_t my_owner, int64_t rows) {
  TORCH_CHECK(expert_of_entry.is_cuda() && expert_of_entry.scalar_type() == torch::kInt32 && expert_of_entry.is_contiguous(), "expert_of_entry: int32");
  TORCH_CHECK(num_experts >= 1 && num_experts <= kMaxLocal && per_owner >= 1 && num_experts % per_owner == 0, "between 1 and 256 experts, evenly split over the owners");
  TORCH_CHECK(my_owner >= 0 && my_owner < num_experts / per_owner, "owner index out of range");
  TORCH_CHECK(rows > 0 && rows % kTile == 0, "rows must be a positive multiple of 128");
  const c10::cuda::CUDAGuard guard(expert_of_entry.device());
  const int64_t entries = expert_of_entry.numel();
  auto opts = expert_of_entry.options();
  Tensor dest_row = torch::empty({entries}, opts);
  Tensor global_row = torch::empty({entries}, opts);
  Tensor src_entry = torch::empty({rows}, opts);
  Tensor tile_expert = torch::empty({rows / kTile}, opts);
  Tensor padded_offsets = torch::empty({per_owner + 1}, opts);
  Tensor dropped = torch::zeros({1}, opts);
  const int blocks = (int)std::max<int64_t>(1, (entries + kChunk - 1) / kChunk);
  Tensor counts = torch::empty({blocks, num_experts}, opts);
  cudaStream_t stream = cur_stream();
  check_cuda(cudaMemsetAsync(src_entry.data_ptr(), 0xFF, (size_t)rows * sizeof(int), stream), "src_entry memset");
  layout_count_kernel<<<blocks, kThreads, 0, stream>>>(expert_of_entry.data_ptr<int>(), (int)entries, 0, (int)num_experts, counts.data_ptr<int>());
  layout_scan_group_kernel<<<1, kThreads, 0, stream>>>(counts.data_ptr<int>(), blocks, (int)num_experts, (int)per_owner, (int)my_owner, (int)rows,
                                                       padded_offsets.data_ptr<int>(), tile_expert.data_ptr<int>());
  layout_place_group_kernel<<<blocks, kThreads, 0, stream>>>(expert_of_entry.data_ptr<int>(), (int)entries, (int)num_experts, (int)per_owner,
                                                             (int)my_owner, counts.data_ptr<int>(), (int)rows, dest_row.data_ptr<int>(),
                                                             src_entry.data_ptr<int>(), global_row.data_ptr<int>(), dropped.data_ptr<int>());
  count_launch(3);
  check_cuda(cudaGetLastError(), "moe_layout_group launch");
  return {dest_row, src_entry, tile_expert, padded_offsets, dropped, global_row};
}

}  // namespace

void register_moe_layout(py::module_& m) {
  m.def("moe_layout", &moe_layout);
  m.def("moe_layout_group", &moe_layout_group);
}

}  // namespace b200
