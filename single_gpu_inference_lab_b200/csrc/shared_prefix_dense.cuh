// Dense shared-prefix pass on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// When every request of a batch attends the same paged prefix (same physical pages in every
// block-table row), the (request, query head) rows of one kv head form a dense matrix:
// 64 requests x 8 heads = 512 rows against the same K/V.  One CTA takes 128 of those rows
// (M = 128), one kv head and one chunk of 256 prefix tokens:
//
//   S[128 x 256] = Q[128 x 128] K^T        tcgen05.mma kind::f16, accumulator in TMEM columns 0..255
//   softmax row-wise, one thread per row (TMEM lane), no shuffles; P (f16) goes to shared memory
//   O[128 x 128] = P[128 x 256] V          tcgen05.mma, accumulator in TMEM columns 256..383
//
// K and V are e4m3 in HBM; the CTA converts its 256 tokens to f16 (exact) while staging them
// as 128-byte-swizzled token rows: K is read as a K-major operand of the first product, V as an
// MN-major operand of the second (head dim contiguous), so nothing is transposed.  A whole chunk is one softmax
// tile, so there is no running maximum and nothing in TMEM is ever rescaled.  The CTA writes
// (o, m, l) of its rows into slot `chunk` of the ordinary split-KV workspace; the suffix pass
// (the generic kernel with kv_start = prefix length) fills the slots after them and the usual
// merge kernel finishes.
//
// Reference counterpart: _shared_paged_prefix_gqa_partial_kernel (tl.dot over BLOCK_M <= 8
// rows x 128 tokens), src/l20_stack/ops/triton_decode_attention.py:704-813.
#pragma once

#include "paged_decode_kernels.cuh"
#include "shared_prefix_groups.cuh"

namespace pfd {

constexpr int kPrefixChunk = 256;  // prefix tokens per CTA
constexpr int kPrefixRows = 128;   // (request, head) rows per CTA
constexpr int kErrUmmaTimeout = 3;

// ---- tcgen05 / TMEM primitives ---------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand in the canonical 128-byte-swizzled
// layout: rows of 64 f16 (128 bytes), 8 rows per 1 KiB atom, atoms stacked along M/N
// (stride-dimension byte offset 1024).  `addr` is the byte address of the first element of
// the 16-element K slice to multiply (a multiple of 32 bytes inside the row).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);       // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                      // leading-dimension byte offset (unused here), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;            // stride-dimension byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                      // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                      // layout type: 128-byte swizzle
  return d;
}
// Descriptor of an MN-major operand (the N index is contiguous in shared memory) in the canonical
// 128-byte-swizzled layout: every K index is a 128-byte row of 64 consecutive N elements, 8 rows
// per 1 KiB atom; atoms of consecutive K groups are 1 KiB apart (stride-dimension offset), blocks
// of 64 N elements `n_block_bytes` apart (leading-dimension offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t addr, uint32_t n_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((n_block_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: f16 x f16 -> f32, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t umma_idesc_f16(int m, int n, bool b_mn_major = false) {
  return (1u << 4)                 // accumulator format f32
         | (0u << 7) | (0u << 10)  // A and B are f16
         | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {  // one thread
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {  // one thread
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int t = 0; t < 32; ++t) v[t] = __uint_as_float(r[t]);
}

// 128 consecutive fp32 columns of this thread's TMEM lane: four loads in flight, one wait.
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld128(uint32_t taddr, float (&v)[128]) {
  uint32_t r[4][32];
#pragma unroll
  for (int q = 0; q < 4; ++q) tmem_ld32_nowait(taddr + 32 * q, r[q]);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int t = 0; t < 32; ++t) v[32 * q + t] = __uint_as_float(r[q][t]);
}

// Byte offset of the 16-byte chunk `c8` (8 f16) of row `row` inside one k-block
// ([rows][64 f16], 128-byte swizzle, block base 1 KiB aligned).
__device__ __forceinline__ uint32_t sw128_chunk(int row, int c8) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((c8 ^ (row & 7)) << 4));
}

// 16 e4m3 bytes -> 16 f16 (two 16-byte chunks)
__device__ __forceinline__ void cvt16_e4m3_f16(const uint4& in, uint4& lo, uint4& hi) {
  lo.x = cvt_e4m3x2_to_f16x2(in.x); lo.y = cvt_e4m3x2_to_f16x2(in.x >> 16);
  lo.z = cvt_e4m3x2_to_f16x2(in.y); lo.w = cvt_e4m3x2_to_f16x2(in.y >> 16);
  hi.x = cvt_e4m3x2_to_f16x2(in.z); hi.y = cvt_e4m3x2_to_f16x2(in.z >> 16);
  hi.z = cvt_e4m3x2_to_f16x2(in.w); hi.w = cvt_e4m3x2_to_f16x2(in.w >> 16);
}

__device__ __forceinline__ void sts_16(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((uint16_t)v) : "memory");
}

struct PrefixParams {
  int32_t prefix_len;   // tokens shared by every request (multiple of 16)
  int32_t batch;
  // Grouped form: the groups buffer of the grouping kernels (shared_prefix_groups.cuh) and its
  // geometry.  grid = (prefix chunks x kv heads, tile slots); the (group, 128-row tile) pairs of
  // the device-side table are numbered in group order and the CTAs of a column take the numbers
  // blockIdx.y, blockIdx.y + gridDim.y, ... in turns, so any number of slots covers the table.
  const int32_t* groups;
  int32_t groups_batch, max_groups;
  int32_t* status;
  unsigned long long wait_limit_ns;  // after this long a wait for the tensor cores gives up and sets the error word
  unsigned long long* phase_times;  // [grid][8] nanosecond stamps; read only in builds with PFD_PHASE_STAMPS
};

// Tuning aid, compiled in only with -DPFD_PHASE_STAMPS.
__device__ __forceinline__ void prefix_mark(const PrefixParams& pp, int k) {
#ifdef PFD_PHASE_STAMPS
  if (pp.phase_times != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const size_t cta = blockIdx.x + gridDim.x * (blockIdx.y + (size_t)gridDim.y * blockIdx.z);
    pp.phase_times[cta * 8 + k] = t;
    if (k == 0) { unsigned r; asm volatile("mov.u32 %0, %%smid;" : "=r"(r)); pp.phase_times[cta * 8 + 7] = r + 1; }
  }
#else
  (void)pp; (void)k;
#endif
}

// grid = (prefix chunks, 128-row tiles, kv heads), block = 512 threads, 1 CTA per SM
// (grouped form: see PrefixParams).
// Warp w works on TMEM lanes (= rows) 32 * (w % 4) .. +31, the only ones it may address, and on
// column group w / 4 of whatever is being read: with 16 warps the staging, the softmax and the
// stores around the two MMAs are spread over all four schedulers four warps deep.
// SLIM caps the kernel at 80 registers per thread (128 otherwise; the cap costs about 1 us of the
// pass).  Registers are handed out per SM sub-partition (16 K each): four warps of this CTA at 80
// registers leave 6144 there, one warp of up to 192 registers -- the two-warp instantiation of
// the suffix kernel uses 165 -- and with the largest shared-memory carve-out two 18 KB CTAs of
// that kind fit beside the 166 KB of this one: the suffix pass then runs on the same SMs WHILE
// this pass runs instead of after it.  (At 126 registers nothing above 32 registers per thread
// fits beside this CTA; without the carve-out request nothing at all, whatever the registers.)
template <bool QBF16, bool SLIM>
__global__ void __maxnreg__(SLIM ? 80 : 128)
shared_prefix_dense_kernel(const KernelParams p, const PrefixParams pp) {
  constexpr int D = 128;
  constexpr uint32_t kQBytes = kPrefixRows * D * 2;         // 32 KiB: 2 k-blocks of [128][64]
  constexpr uint32_t kKBytes = kPrefixChunk * D * 2;        // 64 KiB: 2 k-blocks of [256][64]; later P: 4 x [128][64]; later O rows
  constexpr uint32_t kVBytes = D * kPrefixChunk * 2;        // 64 KiB: 2 d-blocks of [256 tokens][64]
  int chunk = blockIdx.x, mtile = blockIdx.y;
  int kvh = blockIdx.z;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int qd = warp & 3, cg = warp >> 2;  // TMEM lane quarter, column group
  const int row = 32 * qd + lane;           // this thread's (request, head) row of the tile
  pdl_launch_dependents();
  prefix_mark(pp, 0);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sq = base, sk = base + kQBytes, sv = sk + kKBytes;
  const uint32_t bars = sv + kVBytes;       // two mbarriers
  const uint32_t tslot = bars + 16;         // TMEM base address written by tcgen05.alloc
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tslot_ptr = reinterpret_cast<volatile uint32_t*>(gen + kQBytes + kKBytes + kVBytes + 16);
  float* red = reinterpret_cast<float*>(gen + kQBytes + kKBytes + kVBytes + 32);  // [2][4][128] row partials

  // Grouped form: the grid has as many tile slots as the rows of the batch fill; the groups'
  // ragged last tiles can make a few more, which the CTAs of the first slots take in a second
  // turn (tiles done so far = `turns`, the parity the two mbarriers are waited on).  The other
  // form has one tile per CTA.
  int turns = 0;
  uint32_t tmem = 0;
  bool ok = true;
  for (int slot0 = blockIdx.y;; slot0 += gridDim.y) {
    // Which requests, which prefix: the whole batch and pp.prefix_len, or one group of the table.
    int prefix_len = pp.prefix_len, n_req = pp.batch, page_row = 0;
    const int32_t* req_list = nullptr;  // request index of the group's i-th member
    if (pp.groups == nullptr) {
      if (turns > 0) break;
    } else {
      const int B = pp.groups_batch, G = pp.max_groups;
      const int32_t* offs = pp.groups + groups_offsets_off(B);
      // Group of tile slot `slot0`.  Up to 8 groups: all offsets and prefix lengths are fetched at
      // once (offsets of unused groups equal the total, i.e. no tiles), so the lookup costs one
      // round trip to L2 instead of one per dependent step.
      constexpr int kFast = 8;
      int slot = slot0, g = 0, first = 0, members = 0, group_prefix = 0;
      if (G <= kFast) {
        int o[kFast + 1], pl[kFast];
#pragma unroll
        for (int i = 0; i <= kFast; ++i) o[i] = __ldg(offs + min(i, G));
#pragma unroll
        for (int i = 0; i < kFast; ++i) pl[i] = __ldg(pp.groups + groups_prefix_off(B, G) + min(i, G - 1));
        bool found = false;
#pragma unroll
        for (int i = 0; i < kFast; ++i) {
          const int tiles = ((o[i + 1] - o[i]) * p.group + kPrefixRows - 1) / kPrefixRows;
          if (!found && slot < tiles) { found = true; g = i; first = o[i]; members = o[i + 1] - o[i]; group_prefix = pl[i]; }
          if (!found) slot -= tiles;
        }
        if (!found) break;
      } else {
        const int n_groups = min(__ldg(pp.groups + 3), G);
        for (; g < n_groups; ++g) {
          const int tiles = ((__ldg(offs + g + 1) - __ldg(offs + g)) * p.group + kPrefixRows - 1) / kPrefixRows;
          if (slot < tiles) break;
          slot -= tiles;
        }
        if (g >= n_groups) break;
        first = __ldg(offs + g);
        members = __ldg(offs + g + 1) - first;
        group_prefix = __ldg(pp.groups + groups_prefix_off(B, G) + g);
      }
      mtile = slot;
      chunk = blockIdx.x / p.num_kv_heads;
      kvh = blockIdx.x % p.num_kv_heads;
      prefix_len = min(group_prefix & ~15, pp.prefix_len);  // (pp.prefix_len: the cap)
      if (chunk * kPrefixChunk >= prefix_len) continue;
      req_list = pp.groups + groups_rows_off(B, G) + first;
      n_req = members;
      page_row = __ldg(req_list);  // any member's block-table row names the prefix pages
    }

    if (turns == 0) {
      if (t == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      }
      if (warp == 0) tmem_alloc(tslot, 512);
    }
    const uint32_t parity = turns & 1;
    const int tok_lo = chunk * kPrefixChunk;
    const int tok_hi = min(tok_lo + kPrefixChunk, prefix_len);

    // ---- K and V chunk: warp w stages page w of the chunk (16 tokens); per load instruction its
    // lanes cover four whole 128-byte token rows (lane = 8 * token + 16-byte group), so every
    // sector that is fetched is used at once -- with the whole-SM shared-memory carve-out the L1
    // is too small to keep half-used lines until the thread's next load comes back for them
    const int e16 = lane & 7;
    uint4 kin[4], vin[4];
    {
      const bool live = tok_lo + kPage * warp < tok_hi;  // (the prefix ends on a page boundary)
      int64_t phys = 0;
      if (live) phys = page_of(p.block_table, p.bt_stride_b, page_row, tok_lo / kPage + warp);
      const uint8_t* kpage = p.key_cache + phys * p.k_stride_page + (int64_t)kvh * p.k_stride_head;
      const uint8_t* vpage = p.value_cache + phys * p.v_stride_page + (int64_t)kvh * p.v_stride_head;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tp = 4 * c + (lane >> 3);  // token of the page
        kin[c] = vin[c] = make_uint4(0u, 0u, 0u, 0u);
        if (live) {
          kin[c] = __ldg(reinterpret_cast<const uint4*>(kpage + (int64_t)tp * p.k_stride_token) + e16);
          vin[c] = __ldg(reinterpret_cast<const uint4*>(vpage + (int64_t)tp * p.v_stride_token) + e16);
        }
      }
    }
    // ---- Q tile.  This thread's own row (TMEM lane) of the tile, for the softmax and the stores:
    const int row_g = mtile * kPrefixRows + row;
    const int head = row_g % p.group;
    const bool row_live = row_g / p.group < n_req;
    const int b = !row_live ? 0 : (req_list != nullptr ? __ldg(req_list + row_g / p.group) : row_g / p.group);
    // Staging: warp w takes rows 8w .. 8w+7, two whole 256-byte rows per load instruction
    // (lane = 16 * row + 16-byte chunk), fully used sectors as for K and V.
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = 8 * warp + 2 * it + (lane >> 4), c = lane & 15;
      const int rg = mtile * kPrefixRows + r;
      const int req = rg / p.group;
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (req < n_req) {
        const int rb = req_list != nullptr ? __ldg(req_list + req) : req;
        const uint16_t* q = reinterpret_cast<const uint16_t*>(p.query) + (int64_t)rb * p.q_stride_b +
                            (int64_t)(kvh * p.group + rg % p.group) * p.q_stride_h;
        x = __ldg(reinterpret_cast<const uint4*>(q) + c);
      }
      if constexpr (QBF16) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
          w[e] = pack_f16x2(__bfloat162float(v.x), __bfloat162float(v.y));
        }
      }
      sts_16(sq + (c >> 3) * (kPrefixRows * 128) + sw128_chunk(r, c & 7), x);
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {  // 16 bytes = 16 head-dim elements at a time
      const int tr = kPage * warp + 4 * cc + (lane >> 3);  // token row of the chunk
      const int c = e16;
      uint4 lo, hi;
      cvt16_e4m3_f16(kin[cc], lo, hi);
      // K: row = token, k = d; elements 16c .. 16c+15 are chunks 2c, 2c+1 of k-block (c / 4)
      const uint32_t kb = sk + (c >> 2) * (kPrefixChunk * 128);
      sts_16(kb + sw128_chunk(tr, (2 * c) & 7), lo);
      sts_16(kb + sw128_chunk(tr, (2 * c + 1) & 7), hi);
      // V: the same token-major rows (two blocks of 64 head-dim elements); the second MMA reads
      // them as an MN-major operand, so no transposition is needed
      cvt16_e4m3_f16(vin[cc], lo, hi);
      const uint32_t vb = sv + (c >> 2) * (kPrefixChunk * 128);
      sts_16(vb + sw128_chunk(tr, (2 * c) & 7), lo);
      sts_16(vb + sw128_chunk(tr, (2 * c + 1) & 7), hi);
    }
    // generic-proxy writes -> visible to the tensor core's (async proxy) reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    tmem = *tslot_ptr;
    prefix_mark(pp, 1);  // operands staged

    // ---- S = Q K^T : M 128, N 256, K 128 = 2 k-blocks x 4 slices of 16
    if (t == 0) {
      const uint32_t idesc = umma_idesc_f16(128, 256);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int s = 0; s < 4; ++s)
          umma_f16(tmem, umma_desc_k_sw128(sq + kb * (kPrefixRows * 128) + 32 * s),
                   umma_desc_k_sw128(sk + kb * (kPrefixChunk * 128) + 32 * s), idesc, (kb | s) ? 1u : 0u);
      umma_commit(bars);
    }
    ok = mbar_wait_bounded(bars, parity, pp.wait_limit_ns) && ok;
    tc_fence_after_sync();
    prefix_mark(pp, 2);  // S ready

    // ---- softmax: thread (row, cg) holds the row's scores of tokens [64 cg, 64 cg + 64)
    const float ks = p.k_scale_ph ? __ldg(p.k_scale_ph + kvh) : p.k_scale;
    const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + kvh) : p.v_scale;
    const float scale_log2 = ks * p.sm_scale * kLog2e;
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16);  // this warp's 32 TMEM lanes
    const int n_live = tok_hi - tok_lo;
    float sc[64];
    {
      uint32_t r0[32], r1[32];
      tmem_ld32_nowait(lane_addr + 64 * cg, r0);
      tmem_ld32_nowait(lane_addr + 64 * cg + 32, r1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int e = 0; e < 32; ++e) { sc[e] = __uint_as_float(r0[e]); sc[32 + e] = __uint_as_float(r1[e]); }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < 64; ++e)
      if (64 * cg + e < n_live) mx = fmaxf(mx, sc[e]);
    red[cg * 128 + row] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[row], red[128 + row]), fmaxf(red[256 + row], red[384 + row])) * scale_log2;  // scale > 0
    float lsum = 0.f;
#pragma unroll
    for (int e8 = 0; e8 < 8; ++e8) {
      uint4 out;
      uint32_t* w = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const int i0 = 8 * e8 + e;
        const float p0 = (64 * cg + i0 < n_live) ? exp2f(sc[i0] * scale_log2 - mx) : 0.f;
        const float p1 = (64 * cg + i0 + 1 < n_live) ? exp2f(sc[i0 + 1] * scale_log2 - mx) : 0.f;
        lsum += p0 + p1;
        w[e >> 1] = pack_f16x2(p0, p1);
      }
      // P: row = row, k = token 64 cg + 8 e8 ..: chunk e8 of k-block cg
      sts_16(sk + cg * (kPrefixRows * 128) + sw128_chunk(row, e8), out);
    }
    red[512 + cg * 128 + row] = lsum;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    lsum = red[512 + row] + red[640 + row] + red[768 + row] + red[896 + row];

    prefix_mark(pp, 3);  // P written
    // ---- O = P V : M 128, N 128, K 256 = 16 slices of 16 tokens.  A = P (K-major: 4 k-blocks of
    // 64 tokens), B = V (MN-major: 16 tokens = two 1 KiB atoms, d blocks 32 KiB apart)
    if (t == 0) {
      const uint32_t idesc = umma_idesc_f16(128, 128, true);
#pragma unroll
      for (int s = 0; s < 16; ++s)
        umma_f16(tmem + 256, umma_desc_k_sw128(sk + (s >> 2) * (kPrefixRows * 128) + 32 * (s & 3)),
                 umma_desc_mn_sw128(sv + 2048 * s, kPrefixChunk * 128), idesc, s ? 1u : 0u);
      umma_commit(bars + 8);
    }
    ok = mbar_wait_bounded(bars + 8, parity, pp.wait_limit_ns) && ok;
    tc_fence_after_sync();
    prefix_mark(pp, 4);  // O ready

    // ---- (o, m, l) of the rows into slot `chunk` of the workspace.  Thread (row, cg) parks
    // columns [32 cg, +32) of its row in shared memory (16-byte chunks XOR-swizzled by the row);
    // then every warp writes whole rows, 32 lanes x 16 bytes = one contiguous 512-byte row per store.
    {
      float v[32];
      tmem_ld32(lane_addr + 256 + 32 * cg, v);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        sts_16(sk + row * 512 + (((8 * cg + c) ^ (row & 31)) << 4),
               make_uint4(__float_as_uint(v[4 * c] * vs), __float_as_uint(v[4 * c + 1] * vs),
                          __float_as_uint(v[4 * c + 2] * vs), __float_as_uint(v[4 * c + 3] * vs)));
      if (row_live && cg == 0) {
        const int64_t pidx = (int64_t)b * p.partial_stride_b + (int64_t)(kvh * p.group + head) * p.partial_stride_h +
                             (int64_t)chunk * p.partial_stride_s;
        p.partial_max[pidx] = mx * kLn2;
        p.partial_sum[pidx] = lsum;
      }
      __syncthreads();
      for (int r = 0; r < 8; ++r) {
        const int orow = warp * 8 + r;
        const int rg = mtile * kPrefixRows + orow;
        const int rh = rg % p.group;
        if (rg / p.group >= n_req) break;
        const int rb = req_list != nullptr ? __ldg(req_list + rg / p.group) : rg / p.group;
        const uint4 x = lds_16(sk + orow * 512 + ((lane ^ (orow & 31)) << 4));
        const int64_t pidx = (int64_t)rb * p.partial_stride_b + (int64_t)(kvh * p.group + rh) * p.partial_stride_h +
                             (int64_t)chunk * p.partial_stride_s;
        reinterpret_cast<uint4*>(reinterpret_cast<float*>(p.partial_output) + pidx * D)[lane] = x;
      }
    }
    prefix_mark(pp, 5);  // stored
    ++turns;
    // the next tile's staging overwrites what the stores above read, and its MMAs the accumulators
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
  }
  if (turns == 0) return;
  if (!ok && t == 0) atomicExch(pp.status, kErrUmmaTimeout);
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace pfd
