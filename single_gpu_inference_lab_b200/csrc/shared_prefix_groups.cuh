// Device-side detection of shared-prefix groups in a decode batch: which requests begin with the
// same `prefix_len` tokens held in the same pages.  Same key as the reference's host-side
// find_l20_shared_prefix_groups (integrations/vllm/l20_shared_prefix_decode_dispatch.py:41-76:
// prefix length + the prefix's chain of block ids; groups smaller than min_batch and prefixes
// shorter than min_prefix_length are dropped; groups come in the order of their first member),
// but computed where the block table lives, for every group of the batch at once, without a
// host copy: three small kernels once per model step, whose result the grouped decode call of
// every layer reads.
//
//   1. prefix_hash_kernel   one CTA per row: 64-bit position-keyed hash of the row's prefix chain
//   2. prefix_match_kernel  one CTA per row: the first earlier row with equal hash, length AND
//                           chain (verified element by element, so a hash collision costs a
//                           second look, never a wrong group) becomes the row's representative
//   3. prefix_finish_kernel one CTA: numbers the groups, lays out their row lists
//
// Without given prefix lengths the kernels DISCOVER them: rows are keyed on their first
// ceil(min_prefix_len / 16) pages, and a group's prefix is then as long as all of its members
// agree with the representative, in whole pages every member has filled (the reference's trace,
// :245-315, tries one candidate length, floor(min(seq_lens) / 16) * 16, which misses every batch
// whose requests have grown private suffixes of a page or more).
#pragma once

#include <cstdint>

namespace pfd {

constexpr int kGroupsMagic = 0x70666767;
constexpr int kGroupsMaxBatch = 2048;
constexpr int kGroupsHeader = 8;  // magic, batch, max_groups, num_groups, grouped rows, 3 reserved

// Word offsets inside the groups buffer (int32): header, then
//   row_prefix_len[B]  prefix length of the row's group, 0 for a row in no group
//   row_group[B]       index of the row's group, -1 for none
//   group_offsets[G+1] group g's rows are group_rows[group_offsets[g] .. group_offsets[g + 1])
//   group_prefix_len[G]
//   group_rows[B]
//   scratch: rep[B], count[B], lcp[B], hash[2 B]
__host__ __device__ inline int64_t groups_row_prefix_off() { return kGroupsHeader; }
__host__ __device__ inline int64_t groups_row_group_off(int B) { return kGroupsHeader + (int64_t)B; }
__host__ __device__ inline int64_t groups_offsets_off(int B) { return kGroupsHeader + 2LL * B; }
__host__ __device__ inline int64_t groups_prefix_off(int B, int G) { return groups_offsets_off(B) + G + 1; }
__host__ __device__ inline int64_t groups_rows_off(int B, int G) { return groups_prefix_off(B, G) + G; }
__host__ __device__ inline int64_t groups_rep_off(int B, int G) { return groups_rows_off(B, G) + B; }
__host__ __device__ inline int64_t groups_count_off(int B, int G) { return groups_rep_off(B, G) + B; }
__host__ __device__ inline int64_t groups_lcp_off(int B, int G) { return groups_count_off(B, G) + B; }
__host__ __device__ inline int64_t groups_hash_off(int B, int G) { return (groups_lcp_off(B, G) + B + 1) & ~1LL; }
__host__ __device__ inline int64_t groups_words(int B, int G) { return groups_hash_off(B, G) + 2LL * B; }

struct GroupParams {
  const int32_t* block_table;
  int64_t bt_stride_b;
  int32_t bt_cols;
  const int32_t* prefix_lengths;  // per row, or NULL
  int32_t uniform_prefix_len;     // used when prefix_lengths is NULL and this is > 0
  const int32_t* seq_lens;        // else: discover the prefixes (see above); needs the sequence lengths
  int32_t batch, min_batch, min_prefix_len, max_groups;
  int32_t* groups;
};

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__device__ __forceinline__ bool groups_discover(const GroupParams& gp) {
  return gp.prefix_lengths == nullptr && gp.uniform_prefix_len <= 0;
}

// Length of the chain row r is keyed on (0 = the row takes no part).
__device__ __forceinline__ int group_key_len_of(const GroupParams& gp, int r) {
  int len;
  if (groups_discover(gp)) {
    len = (max(gp.min_prefix_len, 16) + 15) / 16 * 16;
    if (gp.seq_lens[r] < len) return 0;
  } else {
    len = gp.prefix_lengths != nullptr ? gp.prefix_lengths[r] : gp.uniform_prefix_len;
  }
  if (len < gp.min_prefix_len || len <= 0) return 0;
  if ((len + 15) / 16 > gp.bt_cols) return 0;  // a prefix the block table cannot hold
  return len;
}

__global__ void __launch_bounds__(256) prefix_hash_kernel(const GroupParams gp) {
  __shared__ unsigned long long sh_h[8];
  const int r = blockIdx.x, B = gp.batch, G = gp.max_groups;
  const int len = group_key_len_of(gp, r);
  const int pages = (len + 15) / 16;
  const int32_t* row = gp.block_table + (int64_t)r * gp.bt_stride_b;
  unsigned long long h = 0;
  for (int i = threadIdx.x; i < pages; i += blockDim.x)
    h += mix64(((uint64_t)(uint32_t)row[i] << 32) ^ (uint64_t)(uint32_t)i ^ 0x9E3779B97F4A7C15ull);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) h += __shfl_xor_sync(0xffffffffu, h, off);
  if ((threadIdx.x & 31) == 0) sh_h[threadIdx.x >> 5] = h;
  __syncthreads();
  if (threadIdx.x == 0) {
    h = 0;
    for (int i = 0; i < 8; ++i) h += sh_h[i];
    h = mix64(h ^ (uint64_t)(uint32_t)len);
    int32_t* g = gp.groups;
    g[groups_hash_off(B, G) + 2 * r] = (int32_t)(uint32_t)h;
    g[groups_hash_off(B, G) + 2 * r + 1] = (int32_t)(uint32_t)(h >> 32);
    g[groups_count_off(B, G) + r] = 0;
    g[groups_row_prefix_off() + r] = len;  // provisional: the finish kernel clears rows left without a group
    // discovery: whole pages this row has filled (and its table can name) bound its group's prefix
    g[groups_lcp_off(B, G) + r] = groups_discover(gp) ? min(gp.seq_lens[r] / 16, gp.bt_cols) : (len + 15) / 16;
    if (r == 0) {
      g[0] = kGroupsMagic; g[1] = B; g[2] = G; g[3] = 0; g[4] = 0; g[5] = g[6] = g[7] = 0;
    }
  }
}

__global__ void __launch_bounds__(256) prefix_match_kernel(const GroupParams gp) {
  __shared__ int sh_min[8];
  __shared__ int sh_same;
  const int r = blockIdx.x, B = gp.batch, G = gp.max_groups;
  int32_t* g = gp.groups;
  const int len = g[groups_row_prefix_off() + r];
  int32_t* rep = g + groups_rep_off(B, G);
  if (len == 0) {
    if (threadIdx.x == 0) rep[r] = -1;
    return;
  }
  const int32_t* hash = g + groups_hash_off(B, G);
  const int32_t* lens = g + groups_row_prefix_off();
  const int h0 = hash[2 * r], h1 = hash[2 * r + 1];
  const int pages = (len + 15) / 16;
  const int32_t* mine = gp.block_table + (int64_t)r * gp.bt_stride_b;
  int found = r;  // its own representative unless an earlier row matches
  for (int start = 0; start < r;) {
    // the first candidate at or after `start`: same hash, same length
    int cand = r;
    for (int i = start + threadIdx.x; i < r; i += blockDim.x)
      if (hash[2 * i] == h0 && hash[2 * i + 1] == h1 && lens[i] == len) { cand = i; break; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, off));
    if ((threadIdx.x & 31) == 0) sh_min[threadIdx.x >> 5] = cand;
    __syncthreads();
    cand = r;
    for (int i = 0; i < 8; ++i) cand = min(cand, sh_min[i]);
    if (cand >= r) break;  // (uniform: every thread computed the same minimum)
    // equal hashes are a strong hint, the chain itself decides
    if (threadIdx.x == 0) sh_same = 1;
    __syncthreads();
    const int32_t* other = gp.block_table + (int64_t)cand * gp.bt_stride_b;
    bool same = true;
    for (int i = threadIdx.x; i < pages && same; i += blockDim.x) same = mine[i] == other[i];
    if (!same) sh_same = 0;
    __syncthreads();
    const bool equal = sh_same != 0;
    __syncthreads();
    if (equal) { found = cand; break; }
    start = cand + 1;
  }
  if (groups_discover(gp) && found != r) {
    // how far beyond the key pages this row agrees with its representative
    const int32_t* other = gp.block_table + (int64_t)found * gp.bt_stride_b;
    const int limit = min(min(gp.seq_lens[r], gp.seq_lens[found]) / 16, gp.bt_cols);
    int first_diff = limit;
    for (int i = pages + threadIdx.x; i < limit; i += blockDim.x)
      if (mine[i] != other[i]) { first_diff = i; break; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) first_diff = min(first_diff, __shfl_xor_sync(0xffffffffu, first_diff, off));
    if ((threadIdx.x & 31) == 0) atomicMin(g + groups_lcp_off(B, G) + found, first_diff);
  }
  if (threadIdx.x == 0) {
    rep[r] = found;
    atomicAdd(g + groups_count_off(B, G) + found, 1);
  }
}

// Block-wide exclusive prefix sum of one value per thread (1024 threads); returns the total too.
__device__ __forceinline__ int block_exclusive_scan(int v, int* sh_warp, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += n;
  }
  if (lane == 31) sh_warp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = sh_warp[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += n;
    }
    sh_warp[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  const int before = warp == 0 ? 0 : sh_warp[warp - 1];
  total = sh_warp[31];
  __syncthreads();
  return before + inc - v;
}

__global__ void __launch_bounds__(1024) prefix_finish_kernel(const GroupParams gp) {
  __shared__ int sh_rep[kGroupsMaxBatch];
  __shared__ int sh_gid[kGroupsMaxBatch];  // group index of a representative row, -1 otherwise
  __shared__ int sh_off[kGroupsMaxBatch];  // first position of a representative's rows in group_rows
  __shared__ int sh_warp[32];
  const int B = gp.batch, G = gp.max_groups;
  int32_t* g = gp.groups;
  const int32_t* rep = g + groups_rep_off(B, G);
  const int32_t* count = g + groups_count_off(B, G);
  const int t = threadIdx.x;
  // two rows per thread: 2 t and 2 t + 1
  int valid[2], cnt[2];
  for (int k = 0; k < 2; ++k) {
    const int r = 2 * t + k;
    valid[k] = 0; cnt[k] = 0;
    if (r < B) {
      sh_rep[r] = rep[r];
      if (rep[r] == r && count[r] >= gp.min_batch) { valid[k] = 1; cnt[k] = count[r]; }
    }
  }
  int total_groups = 0, total_rows = 0;
  const int gbase = block_exclusive_scan(valid[0] + valid[1], sh_warp, total_groups);
  for (int k = 0; k < 2; ++k) {
    const int r = 2 * t + k;
    if (r < B) {
      const int gid = gbase + (k == 1 ? valid[0] : 0);
      const bool keep = valid[k] && gid < G;  // groups beyond the buffer's capacity are left out
      sh_gid[r] = keep ? gid : -1;
      if (!keep) cnt[k] = 0;
    }
  }
  const int obase = block_exclusive_scan(cnt[0] + cnt[1], sh_warp, total_rows);
  for (int k = 0; k < 2; ++k) {
    const int r = 2 * t + k;
    if (r < B) {
      sh_off[r] = obase + (k == 1 ? cnt[0] : 0);
      if (sh_gid[r] >= 0) {
        g[groups_offsets_off(B) + sh_gid[r]] = sh_off[r];
        g[groups_prefix_off(B, G) + sh_gid[r]] =
            groups_discover(gp) ? 16 * g[groups_lcp_off(B, G) + r] : g[groups_row_prefix_off() + r];
      }
    }
  }
  __syncthreads();
  const int ngroups = min(total_groups, G);
  if (t == 0) {
    g[3] = ngroups;
    g[4] = total_rows;
    g[groups_offsets_off(B) + ngroups] = total_rows;
  }
  for (int i = ngroups + 1 + t; i <= G; i += blockDim.x) g[groups_offsets_off(B) + i] = total_rows;
  // every row: its group, its place among the group's rows (members in ascending order)
  for (int r = t; r < B; r += blockDim.x) {
    const int rp = sh_rep[r];
    const int gid = rp >= 0 ? sh_gid[rp] : -1;
    if (gid < 0) {
      g[groups_row_group_off(B) + r] = -1;
      g[groups_row_prefix_off() + r] = 0;
      continue;
    }
    int rank = 0;
    for (int i = rp; i < r; ++i) rank += sh_rep[i] == rp;
    g[groups_row_group_off(B) + r] = gid;
    g[groups_rows_off(B, G) + sh_off[rp] + rank] = r;
    if (groups_discover(gp)) g[groups_row_prefix_off() + r] = 16 * g[groups_lcp_off(B, G) + rp];
  }
}

}  // namespace pfd
