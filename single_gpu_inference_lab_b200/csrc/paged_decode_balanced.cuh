// Balanced, persistent form of the split-KV decode step for head_dim 128 (sm_100a).
//
// Instead of a grid of fixed (sequence, kv head, split) work items, a fixed number of warps
// (eight per SM) share the flattened list of page pairs of all sequences: the warps form
// groups of one warp per kv head, and every group takes an equal contiguous chunk of the list,
// so every warp streams the same number of KV bytes whatever the mix of context lengths, and
// no CTA is launched for a split that does not exist.  The warps of a group read the same pages
// at about the same time, each its own head, which keeps the rows of a page that lie next to
// each other in memory (token-major layout) in one burst of DRAM traffic.  A warp walks the
// sequences its chunk overlaps on its own: no barrier, no shared accumulator, one private TMA
// ring that keeps loading across sequence boundaries.  A sequence that lies inside one chunk
// is finished by that warp (final output rows, or the packed (o, m, l) form); the piece of a
// sequence that straddles chunks goes to the caller's workspace as (o, m, l), into one of the
// two slots every group owns, and the merge kernel behind (programmatic dependent launch)
// combines the pieces.  Both kernels derive the chunking from seq_lens alone, so nothing but
// the pieces themselves passes between them.
//
// Maths per page pair and warp, "heads as columns": S^T = K Q^T and O^T += V^T P^T with
// mma.sync.m16n8k16 (f16 in, f32 accumulate).  Tokens (resp. head-dim rows) fill the 16-row M
// dimension and the <= 8 query heads of the group fill N = 8 exactly, so nothing of the tile is
// padding, O^T needs 32 accumulator registers, and P^T reaches its B-fragment layout with one
// movmatrix per 8 tokens.
#pragma once

#include <type_traits>

#include "paged_decode_kernels.cuh"

namespace pfd {

struct ChunkParams {
  int32_t batch;
  int32_t num_warps;   // warps of the whole grid; the merge kernel is told the same number
  int32_t piece_cost;  // what starting a sequence costs a warp, in half page pairs
  int32_t* plan;       // device plan written by plan_decode_kernel, or nullptr
};

// How the work is cut.  Cost is counted in half page pairs: sequence b owns the cost range that
// starts at 2 * (pairs before b) + piece_cost * b, first piece_cost units for taking the
// sequence up (query fetch, state reset, output rows), then two units per page pair.  The cost
// axis is cut into `groups` contiguous chunks whose lengths differ by at most one unit, and a
// page pair belongs to the chunk that holds its first unit.  Tiny workloads use fewer groups so
// that no chunk is shorter than kMinChunkCost units (a chunk inside a sequence is never empty).
// (Cutting at page granularity, a pair shared by two chunks that each attend one of its pages,
// balances bytes better but was measured slower: the shared pairs cost both chunks a step.)
constexpr int kMinChunkCost = 8;
struct Chunking {
  int base, rem, groups, piece_cost;
  __device__ __forceinline__ Chunking(int total_pairs, int batch, int max_groups, int cost) : piece_cost(cost) {
    const int total = 2 * total_pairs + cost * batch;
    groups = max(min(max_groups, total / kMinChunkCost), 1);
    base = total / groups;
    rem = total - base * groups;
  }
  __device__ __forceinline__ int start_of(int c) const { return c * base + min(c, rem); }
  __device__ __forceinline__ int chunk_of(int unit) const {
    const int wide = rem * (base + 1);
    return unit < wide ? unit / (base + 1) : rem + (unit - wide) / max(base, 1);
  }
  // first cost unit of pair 0 of sequence b, given the pairs before b
  __device__ __forceinline__ int first_unit(int pairs_before, int b) const {
    return 2 * pairs_before + piece_cost * (b + 1);
  }
};

// Page pairs of a sequence of `len` tokens when attention starts at token `kv_start`: none if
// the sequence ends at or before it (a page that holds only tokens in front of kv_start would
// give a piece without a single live token, hence 0 / 0).
__device__ __forceinline__ int pairs_of(int len, int kv_start) {
  const int pages = len > kv_start ? (len + kPage - 1) / kPage - kv_start / kPage : 0;
  return (pages + 1) >> 1;
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// Running state of one warp for the current segment, NH head tiles of 8 heads.
template <int NH>
struct BalState {
  float o[NH][8][4];  // [head tile][m-tile mt][c]: d = 16i + 2mt + (c>>1), head = 8h + 2j + (c&1)
  float m[NH][2];     // running max (log2 domain) of heads 2j, 2j+1
  float l[NH][2];     // running sum over this thread's tokens only
};

template <int NH>
__device__ __forceinline__ void bal_reset(BalState<NH>& st) {
#pragma unroll
  for (int h = 0; h < NH; ++h) {
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) st.o[h][mt][0] = st.o[h][mt][1] = st.o[h][mt][2] = st.o[h][mt][3] = 0.f;
    st.m[h][0] = st.m[h][1] = -INFINITY;
    st.l[h][0] = st.l[h][1] = 0.f;
  }
}

// Q of head (8h + i) as B-fragments: k-step ks = 4l + w covers d = 16(j+4l) + 4w + {0,1 | 2,3}.
template <bool QBF16, int NH>
__device__ __forceinline__ void bal_load_q(uint32_t (&qb)[NH][8][2], const KernelParams& p, int b,
                                           int kvh, int i, int j) {
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const int head = 8 * h + i;
    const bool live = head < p.group;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(p.query) + (int64_t)b * p.q_stride_b +
                        (int64_t)(kvh * p.group + (live ? head : 0)) * p.q_stride_h;
#pragma unroll
    for (int l = 0; l < 2; ++l) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint2 raw = make_uint2(0u, 0u);
        if (live) raw = __ldg(reinterpret_cast<const uint2*>(q + 16 * (j + 4 * l) + 4 * w));
        if constexpr (QBF16) {
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          raw.x = pack_f16x2(__bfloat162float(a.x), __bfloat162float(a.y));
          raw.y = pack_f16x2(__bfloat162float(c.x), __bfloat162float(c.y));
        }
        qb[h][l * 4 + w][0] = raw.x;
        qb[h][l * 4 + w][1] = raw.y;
      }
    }
  }
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One step = two consecutive pages (32 tokens) of one segment, read from a stage
// [K0][K1][V0][V1] (2 KiB tiles, 128-byte swizzle).  tok0 = token index of page 0's row 0.
template <int NH>
__device__ __forceinline__ void bal_step(BalState<NH>& st, uint32_t stage, const uint32_t (&k_off)[2][2],
                                         const uint32_t (&v_off)[4], const uint32_t (&qb)[NH][8][2],
                                         float scale_log2, int tok0, int lo, int hi, int i, int j) {
  constexpr uint32_t kTile = kPage * 128;
  const bool edge = (tok0 < lo) | (tok0 + 2 * kPage > hi);
  float s[NH][2][4];
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int u = 0; u < 2; ++u) s[h][u][0] = s[h][u][1] = s[h][u][2] = s[h][u][3] = 0.f;
  {
    uint32_t k[2][2][2][4];  // [page][row half][l][word]
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int l = 0; l < 2; ++l) {
          const uint4 x = lds_16(stage + u * kTile + k_off[half][l]);
          k[u][half][l][0] = x.x; k[u][half][l][1] = x.y; k[u][half][l][2] = x.z; k[u][half][l][3] = x.w;
        }
#pragma unroll
    for (int l = 0; l < 2; ++l)
#pragma unroll
      for (int w = 0; w < 4; ++w)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t r0 = k[u][0][l][w], r1 = k[u][1][l][w];
          const uint32_t a0 = cvt_e4m3x2_to_f16x2(r0), a1 = cvt_e4m3x2_to_f16x2(r1);
          const uint32_t a2 = cvt_e4m3x2_to_f16x2(r0 >> 16), a3 = cvt_e4m3x2_to_f16x2(r1 >> 16);
#pragma unroll
          for (int h = 0; h < NH; ++h) mma_16816(s[h][u], a0, a1, a2, a3, qb[h][l * 4 + w][0], qb[h][l * 4 + w][1]);
        }
  }
  // scale + mask: s[h][u][c] is (token 16u + 8(c>>1) + rho(i), head 8h + 2j + (c&1))
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      bool dead = false;
      if (edge) {
        const int tok = tok0 + u * kPage + 8 * (c >> 1) + rho(i);
        dead = (tok < lo) | (tok >= hi);
      }
#pragma unroll
      for (int h = 0; h < NH; ++h) s[h][u][c] = dead ? -INFINITY : s[h][u][c] * scale_log2;
    }
  uint32_t pb[NH][2][2];  // P^T B-fragments [head tile][page][b0|b1]
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    float mx[2], alpha[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float x = fmaxf(fmaxf(s[h][0][e], s[h][0][2 + e]), fmaxf(s[h][1][e], s[h][1][2 + e]));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 8));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 16));
      mx[e] = fmaxf(st.m[h][e], x);
      alpha[e] = exp2f(st.m[h][e] - mx[e]);
      st.m[h][e] = mx[e];
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float p0 = exp2f(s[h][u][0] - mx[0]), p1 = exp2f(s[h][u][1] - mx[1]);
      const float p2 = exp2f(s[h][u][2] - mx[0]), p3 = exp2f(s[h][u][3] - mx[1]);
      sum[0] += p0 + p2;
      sum[1] += p1 + p3;
      // (token row i, heads 2j, 2j+1) -> transpose -> (tokens rho(2j), rho(2j+1); head i)
      pb[h][u][0] = movmatrix_trans(pack_f16x2(p0, p1));
      pb[h][u][1] = movmatrix_trans(pack_f16x2(p2, p3));
    }
    st.l[h][0] = st.l[h][0] * alpha[0] + sum[0];
    st.l[h][1] = st.l[h][1] * alpha[1] + sum[1];
    if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        st.o[h][mt][0] *= alpha[0]; st.o[h][mt][1] *= alpha[1];
        st.o[h][mt][2] *= alpha[0]; st.o[h][mt][3] *= alpha[1];
      }
    }
  }
  // O^T += V^T P^T
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    uint32_t v[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint4 x = lds_16(stage + (2 + u) * kTile + v_off[r]);
      v[r][0] = x.x; v[r][1] = x.y; v[r][2] = x.z; v[r][3] = x.w;
    }
    if (edge) {  // bytes of tokens outside the range may hold anything: 0 * NaN must not happen
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int tok = tok0 + u * kPage + v_row(j, r);
        if (tok < lo || tok >= hi) v[r][0] = v[r][1] = v[r][2] = v[r][3] = 0u;
      }
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t x01 = prmt(v[0][w], v[1][w], 0x5140u), y01 = prmt(v[0][w], v[1][w], 0x7362u);
      const uint32_t x23 = prmt(v[2][w], v[3][w], 0x5140u), y23 = prmt(v[2][w], v[3][w], 0x7362u);
      const uint32_t e0 = cvt_e4m3x2_to_f16x2(x01), e1 = cvt_e4m3x2_to_f16x2(x01 >> 16);
      const uint32_t e2 = cvt_e4m3x2_to_f16x2(x23), e3 = cvt_e4m3x2_to_f16x2(x23 >> 16);
      const uint32_t f0 = cvt_e4m3x2_to_f16x2(y01), f1 = cvt_e4m3x2_to_f16x2(y01 >> 16);
      const uint32_t f2 = cvt_e4m3x2_to_f16x2(y23), f3 = cvt_e4m3x2_to_f16x2(y23 >> 16);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        mma_16816(st.o[h][2 * w], e0, e1, e2, e3, pb[h][u][0], pb[h][u][1]);
        mma_16816(st.o[h][2 * w + 1], f0, f1, f2, f3, pb[h][u][0], pb[h][u][1]);
      }
    }
  }
}

template <bool QBF16>
__device__ __forceinline__ void store_row16(const KernelParams& p, int b, int hq, int d0, const float (&v)[16],
                                            float m_nat, float l, bool write_ml, uint32_t xstep) {
  // 16 consecutive head-dim values of one (sequence, q head) row: final output, packed form, or
  // tagged words into every rank's receive buffer
  if (p.xch_world > 0) {
    for (int dest = 0; dest < p.xch_world; ++dest) {
      unsigned long long* dst = xch_row(p, dest, (int64_t)b * p.num_q_heads + hq, xstep);
#pragma unroll
      for (int t = 0; t < 16; t += 2) xch_store2(dst + d0 + t, v[t], v[t + 1], xstep);
      if (write_ml) xch_store2(dst + 128, m_nat, l, xstep);
    }
  } else if (p.packed_output != nullptr) {
    float* dst = p.packed_output + ((int64_t)b * p.num_q_heads + hq) * 130 + d0;
#pragma unroll
    for (int t = 0; t < 16; t += 2) *reinterpret_cast<float2*>(dst + t) = make_float2(v[t], v[t + 1]);
    if (write_ml) { dst[128 - d0] = m_nat; dst[129 - d0] = l; }
  } else {
    const float inv = 1.f / l;
    uint32_t w[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if constexpr (QBF16) {
        __nv_bfloat162 x = __floats2bfloat162_rn(v[2 * t] * inv, v[2 * t + 1] * inv);
        w[t] = *reinterpret_cast<uint32_t*>(&x);
      } else {
        w[t] = pack_f16x2(v[2 * t] * inv, v[2 * t + 1] * inv);
      }
    }
    uint16_t* dst = reinterpret_cast<uint16_t*>(p.output) + (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h + d0;
    *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    *reinterpret_cast<uint2*>(dst + 4) = make_uint2(w[2], w[3]);
    *reinterpret_cast<uint2*>(dst + 8) = make_uint2(w[4], w[5]);
    *reinterpret_cast<uint2*>(dst + 12) = make_uint2(w[6], w[7]);
  }
}


// ---- 16-bit (fp16 / bf16) K/V caches ---------------------------------------------------------
// Same kernel, other tiles: a (page, head) tile is 16 rows of 256 bytes, staged as two
// 128-byte-swizzled halves of 2 KiB ([d 0..63], [d 64..127]); fragments come from ldmatrix, K
// as it lies (tokens x d), V transposed (d x tokens); no conversion step.  Accumulators are in
// the natural MMA layout: o[mt][c] is d = 16 mt + i + 8 (c >> 1), head 2j + (c & 1).
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma_16816_kv16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack_kv16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 x = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&x);
  } else {
    return pack_f16x2(lo, hi);
  }
}

// Q of head i as B-fragments in natural order: k-step ks covers d = 16 ks + 2j + {0,1 | 8,9}.
__device__ __forceinline__ void kv16_load_q(uint32_t (&qb)[1][8][2], const KernelParams& p, int b, int kvh,
                                            int i, int j) {
  const bool live = i < p.group;
  const uint32_t* q = reinterpret_cast<const uint32_t*>(
      reinterpret_cast<const uint16_t*>(p.query) + (int64_t)b * p.q_stride_b +
      (int64_t)(kvh * p.group + (live ? i : 0)) * p.q_stride_h);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qb[0][ks][0] = live ? __ldg(q + 8 * ks + j) : 0u;
    qb[0][ks][1] = live ? __ldg(q + 8 * ks + 4 + j) : 0u;
  }
}

// One step = two consecutive pages of one sequence, read from a stage [K0][K1][V0][V1] of
// 4 KiB tiles (two swizzled halves each).  tok0 = token index of page 0's row 0.
template <bool BF16>
__device__ __forceinline__ void kv16_step(BalState<1>& st, uint32_t stage, const uint32_t (&qb)[1][8][2],
                                          float scale_log2, int tok0, int lo, int hi, int lane) {
  constexpr uint32_t kTile = 2 * kPage * 128;
  const int i = lane >> 2, j = lane & 3;
  const int mid = lane >> 3, r8 = lane & 7;
  const bool edge = (tok0 < lo) | (tok0 + 2 * kPage > hi);
  float s[2][4];
#pragma unroll
  for (int u = 0; u < 2; ++u) s[u][0] = s[u][1] = s[u][2] = s[u][3] = 0.f;
  {
    // K: matrix `mid` of an x4 load = rows 8 (mid & 1) .., 16-byte chunk 2 ks + (mid >> 1)
    const int row = (mid & 1) * 8 + r8;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int chunk = 2 * ks + (mid >> 1);
      const uint32_t off = (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint32_t a[4];
        ldsm_x4(stage + u * kTile + off, a);
        mma_16816_kv16<BF16>(s[u], a, qb[0][ks][0], qb[0][ks][1]);
      }
    }
  }
  // scale + mask: s[u][c] is (token 16u + 8(c>>1) + i, head 2j + (c&1))
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      bool dead = false;
      if (edge) {
        const int tok = tok0 + u * kPage + 8 * (c >> 1) + i;
        dead = (tok < lo) | (tok >= hi);
      }
      s[u][c] = dead ? -INFINITY : s[u][c] * scale_log2;
    }
  // P^T B-fragments.  bf16 keeps 8 bits of a probability: there P goes in as two bf16 terms
  // (p = hi + lo, 16 bits together) and the PV product takes two MMAs; f16 keeps 11 bits.
  uint32_t pb[2][2], pl[2][2];
  {
    float mx[2], alpha[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float x = fmaxf(fmaxf(s[0][e], s[0][2 + e]), fmaxf(s[1][e], s[1][2 + e]));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 8));
      x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 16));
      mx[e] = fmaxf(st.m[0][e], x);
      alpha[e] = exp2f(st.m[0][e] - mx[e]);
      st.m[0][e] = mx[e];
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float p0 = exp2f(s[u][0] - mx[0]), p1 = exp2f(s[u][1] - mx[1]);
      const float p2 = exp2f(s[u][2] - mx[0]), p3 = exp2f(s[u][3] - mx[1]);
      sum[0] += p0 + p2;
      sum[1] += p1 + p3;
      // (token i, heads 2j, 2j+1) -> transpose -> (tokens 2j, 2j+1; head i)
      pb[u][0] = movmatrix_trans(pack_kv16<BF16>(p0, p1));
      pb[u][1] = movmatrix_trans(pack_kv16<BF16>(p2, p3));
      if constexpr (BF16) {
        const auto hi = [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); };
        pl[u][0] = movmatrix_trans(pack_kv16<true>(p0 - hi(p0), p1 - hi(p1)));
        pl[u][1] = movmatrix_trans(pack_kv16<true>(p2 - hi(p2), p3 - hi(p3)));
      }
    }
    st.l[0][0] = st.l[0][0] * alpha[0] + sum[0];
    st.l[0][1] = st.l[0][1] * alpha[1] + sum[1];
    if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        st.o[0][mt][0] *= alpha[0]; st.o[0][mt][1] *= alpha[1];
        st.o[0][mt][2] *= alpha[0]; st.o[0][mt][3] *= alpha[1];
      }
    }
  }
  // O^T += V^T P^T.  V^T fragments by transposing loads: matrix `mid` = tokens 8 (mid >> 1) ..,
  // chunk 2 mt + (mid & 1); a[0], a[1] hold tokens 2j, 2j+1 and a[2], a[3] tokens 8 + 2j, 9 + 2j.
  {
    const int row = (mid >> 1) * 8 + r8;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      uint32_t keep_lo = 0xffffffffu, keep_hi = 0xffffffffu;  // bytes of tokens outside the range may hold anything
      if (edge) {
        const int t0 = tok0 + u * kPage + 2 * j;
        const auto live = [&](int t) { return (t >= lo) & (t < hi); };
        keep_lo = (live(t0) ? 0x0000ffffu : 0u) | (live(t0 + 1) ? 0xffff0000u : 0u);
        keep_hi = (live(t0 + 8) ? 0x0000ffffu : 0u) | (live(t0 + 9) ? 0xffff0000u : 0u);
      }
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        const int chunk = 2 * mt + (mid & 1);
        const uint32_t off = (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
        uint32_t a[4];
        ldsm_x4_trans(stage + (2 + u) * kTile + off, a);
        if (edge) { a[0] &= keep_lo; a[1] &= keep_lo; a[2] &= keep_hi; a[3] &= keep_hi; }
        mma_16816_kv16<BF16>(st.o[0][mt], a, pb[u][0], pb[u][1]);
        if constexpr (BF16) mma_16816_kv16<true>(st.o[0][mt], a, pl[u][0], pl[u][1]);
      }
    }
  }
}

// One value of a piece into the workspace in its storage type.
__device__ __forceinline__ void store_partial_scalar(void* base, int dtype, int64_t idx, float v) {
  if (dtype == 0) reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == 1) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}

// Workspace row of query head `hq` in slot `which` of warp group `grp` (0: the piece that begins
// the chunk, 1: the piece that ends it).  The workspace is used as a flat array of (o[D], m, l) rows.
__device__ __forceinline__ int64_t chunk_slot_row(int grp, int which, int num_q_heads, int hq) {
  return ((int64_t)(2 * grp + which)) * num_q_heads + hq;
}

// ---- the plan ------------------------------------------------------------------------------
// Everything the chunk kernel derives from seq_lens and block_table alone, computed once per
// model step (the metadata is the same for every layer) by plan_decode_kernel and read by the
// chunk kernel of every layer: the pair prefix sum, each warp group's range of the pair list
// with the page ids of its first 16 pairs (so a warp's first copies leave after one round trip
// to L2), and one arrival counter per (sequence, kv head) that lets the pieces of a cut
// sequence be combined inside the chunk kernel, by the warp whose piece arrives last.
// Layout, in 32-bit words:
//   [0, 16)            header (kPlan* indices below)
//   [16, 16 + B + 1)   pairs before sequence b
//   [.., + B)          sequence lengths
//   groups_off         per group kPlanGroupWords words: P0, P1, mask of those of its first 16 pairs
//                      that end a sequence (hold its last page), 1 reserved, 32 page ids
//   counters_off       B * Hkv arrival counters (page pairs consumed), zero between launches
constexpr int kPlanMagic = 0x70666431;
constexpr int kPlanHeaderWords = 16;
constexpr int kPlanGroupWords = 36;
enum { kPlanWMagic = 0, kPlanWBatch, kPlanWKvStart, kPlanWKvHeads, kPlanWMaxGroups, kPlanWPieceCost, kPlanWTotal,
       kPlanWIndptr };
__host__ __device__ inline int64_t plan_groups_off(int batch) { return (kPlanHeaderWords + 2 * (int64_t)batch + 1 + 3) & ~3LL; }
__host__ __device__ inline int64_t plan_counters_off(int batch, int max_groups) {
  return plan_groups_off(batch) + (int64_t)max_groups * kPlanGroupWords;
}
__host__ __device__ inline int64_t plan_words(int batch, int max_groups, int num_kv_heads) {
  return plan_counters_off(batch, max_groups) + (int64_t)batch * num_kv_heads;
}

constexpr int kErrPlanMismatch = 2;

// What a warp needs to walk the flattened pair list: the prefix sum and the lengths (shared
// memory), the geometry, and the chunking.
struct PairList {
  const int32_t* prefix;  // [B + 1]
  const int32_t* lens;    // [B]
  int B, page_first, kv_start;
  // Sequence that holds pair g of the list (0 <= g < total): largest b with prefix[b] <= g.
  __device__ __forceinline__ int seq_of(int g) const {
    int lo_b = 0, hi_b = B;
    while (hi_b - lo_b > 1) {
      const int mid = (lo_b + hi_b) >> 1;
      if (prefix[mid] <= g) lo_b = mid; else hi_b = mid;
    }
    return lo_b;
  }
  // Pairs whose first cost unit lies before cost position c.
  __device__ __forceinline__ int pairs_before(const Chunking& chunks, int c) const {
    const int total = prefix[B];
    if (c >= 2 * total + chunks.piece_cost * B) return total;
    int lo_b = 0, hi_b = B;  // largest b whose cost range starts at or before c
    while (hi_b - lo_b > 1) {
      const int mid = (lo_b + hi_b) >> 1;
      if (2 * prefix[mid] + chunks.piece_cost * mid <= c) lo_b = mid; else hi_b = mid;
    }
    const int off = c - chunks.first_unit(prefix[lo_b], lo_b);  // units into the pairs of lo_b
    return prefix[lo_b] + min(max((off + 1) >> 1, 0), prefix[lo_b + 1] - prefix[lo_b]);
  }
};

// The pairs a chunk steps through: [P0, P1) of the flattened pair list.
struct ChunkRange {
  int P0, P1;
};
__device__ __forceinline__ ChunkRange chunk_range(const PairList& list, const Chunking& chunks, int grp) {
  ChunkRange r;
  const int total = list.prefix[list.B];
  if (grp >= chunks.groups) {
    r.P0 = r.P1 = total;
    return r;
  }
  r.P0 = list.pairs_before(chunks, chunks.start_of(grp));
  r.P1 = list.pairs_before(chunks, chunks.start_of(grp + 1));
  return r;
}

// Page ids of 16 consecutive pairs of a chunk, one page per lane (lane 2t + u holds page u of
// pair P0 + base_t + t, -1 if there is none).
__device__ __forceinline__ int32_t fetch_ids(const PairList& list, const KernelParams& p, const ChunkRange& cr,
                                             int base_t, int lane) {
  int32_t phys = -1;
  const int g = cr.P0 + base_t + (lane >> 1);
  if (g < cr.P1) {
    const int b = list.seq_of(g);
    const int page = list.page_first + 2 * (g - list.prefix[b]) + (lane & 1);
    if (page <= (list.lens[b] - 1) / kPage)
      phys = p.page_indptr ? __ldg(p.block_table + __ldg(p.page_indptr + b) + page)
                           : page_of(p.block_table, p.bt_stride_b, b, page);
  }
  return phys;
}

// Pairs per sequence and their exclusive prefix sum into shared memory, by all NT threads of the
// CTA (every CTA computes the same).  Ends with a CTA-wide barrier.
template <int NT>
__device__ __forceinline__ void scan_pairs(const int32_t* __restrict__ seq_lens, int B, int kv_start,
                                           int32_t* sm_scan, int32_t* prefix, int32_t* lens) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (B + NT - 1) / NT;
  const int b0 = threadIdx.x * per;
  int local = 0;
  for (int q = 0; q < per; ++q) {
    const int b = b0 + q;
    if (b < B) {
      const int len = seq_lens[b];
      lens[b] = len;
      local += pairs_of(len, kv_start);
    }
  }
  int incl = local;  // inclusive scan over the CTA's threads
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int x = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += x;
  }
  if (lane == 31) sm_scan[warp] = incl;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += sm_scan[w];
  int run = before + incl - local;
  for (int q = 0; q < per; ++q) {
    const int b = b0 + q;
    if (b < B) {
      prefix[b] = run;
      run += pairs_of(lens[b], kv_start);
    }
  }
  if (threadIdx.x == NT - 1) prefix[B] = before + incl;
  __syncthreads();
}

struct PlanParams {
  const int32_t* __restrict__ seq_lens;
  const int32_t* __restrict__ block_table;
  const int32_t* __restrict__ page_indptr;
  int64_t bt_stride_b;
  int32_t batch, kv_start, num_kv_heads, max_groups, piece_cost;
  int32_t* plan;
};

// Writes the plan.  grid = a few CTAs (each repeats the scan, then takes every gridDim-th warp
// group), block = 1024 threads.  Needs batch <= kPlanMaxBatch.
constexpr int kPlanMaxBatch = 2048;
__global__ void __launch_bounds__(1024) plan_decode_kernel(const PlanParams pp) {
  constexpr int NT = 1024;
  __shared__ int32_t sm_scan[NT / 32];
  __shared__ int32_t prefix[kPlanMaxBatch + 1];
  __shared__ int32_t lens[kPlanMaxBatch];
  const int B = pp.batch;
  scan_pairs<NT>(pp.seq_lens, B, pp.kv_start, sm_scan, prefix, lens);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* plan = pp.plan;
  if (blockIdx.x == 0) {
    if (threadIdx.x < kPlanHeaderWords) {
      int32_t v = 0;
      switch (threadIdx.x) {
        case kPlanWMagic: v = kPlanMagic; break;
        case kPlanWBatch: v = B; break;
        case kPlanWKvStart: v = pp.kv_start; break;
        case kPlanWKvHeads: v = pp.num_kv_heads; break;
        case kPlanWMaxGroups: v = pp.max_groups; break;
        case kPlanWPieceCost: v = pp.piece_cost; break;
        case kPlanWTotal: v = prefix[B]; break;
        case kPlanWIndptr: v = pp.page_indptr != nullptr ? 1 : 0; break;
        default: break;
      }
      plan[threadIdx.x] = v;
    }
    for (int x = threadIdx.x; x <= B; x += NT) plan[kPlanHeaderWords + x] = prefix[x];
    for (int x = threadIdx.x; x < B; x += NT) plan[kPlanHeaderWords + B + 1 + x] = lens[x];
  }
  {
    int32_t* counters = plan + plan_counters_off(B, pp.max_groups);
    const int n = B * pp.num_kv_heads;
    for (int x = blockIdx.x * NT + threadIdx.x; x < n; x += gridDim.x * NT) counters[x] = 0;
  }
  KernelParams kp{};  // only what fetch_ids reads
  kp.block_table = pp.block_table;
  kp.page_indptr = pp.page_indptr;
  kp.bt_stride_b = pp.bt_stride_b;
  const PairList list{prefix, lens, B, pp.kv_start / kPage, pp.kv_start};
  const Chunking chunks(prefix[B], B, max(pp.max_groups, 1), pp.piece_cost);
  for (int grp = blockIdx.x * (NT / 32) + warp; grp < pp.max_groups; grp += gridDim.x * (NT / 32)) {
    const ChunkRange cr = chunk_range(list, chunks, grp);
    const int32_t id = fetch_ids(list, kp, cr, 0, lane);
    int32_t* gw = plan + plan_groups_off(B) + (int64_t)grp * kPlanGroupWords;
    // which of the group's first 16 pairs end their sequence: a decode step's cache append writes
    // there and nowhere else, so these are the only pairs that must wait for it (early_kv)
    const int gpair = cr.P0 + lane;
    const bool last_of_seq = lane < 16 && gpair < cr.P1 && gpair + 1 == prefix[list.seq_of(gpair) + 1];
    const unsigned ends = __ballot_sync(0xffffffffu, last_of_seq);
    if (lane == 0) { gw[0] = cr.P0; gw[1] = cr.P1; gw[2] = (int32_t)ends; gw[3] = 0; }
    gw[4 + lane] = id;
  }
}

// In-kernel LSE merge of the pieces of one (sequence, kv head), run by the warp whose piece
// arrived last: rows (query head h of the group, piece k) are fetched 32 at a time (one 512-byte
// row per load instruction, all 32 in flight together) from the workspace, which the pieces'
// writers left in L2, and folded head by head with a running maximum.  Same maths as
// _paged_split_kv_reduce (integrations/vllm/l20_paged_split_kv.py:459-488).
// Kept out of line on purpose: with registers of its own the 32 loads of a batch stay in
// flight together; inlined into the streaming loop they were issued one after the other.
struct MergeJob {
  const float* po;   // workspace rows (o), maxima, sums
  const float* pm;
  const float* pl;
  void* output;
  float* packed;
  int64_t o_stride_b, o_stride_h;
  int32_t num_q_heads, hq0, group;  // hq0: first query head of the kv head
  int32_t ns, w_first, which0;      // pieces, chunk of piece 0, slot of piece 0 in its chunk
  int32_t b;
#ifdef PFD_BOUNDS_CHECK
  int64_t ws_rows;                  // self-checking builds: rows of the workspace
  unsigned long long* report;
#endif
};

template <bool QBF16, bool PACKED>
__device__ __noinline__ void merge_pieces_of_sequence(const MergeJob j, const int lane) {
  constexpr int D = 128, RB = 32;
  const int ns = j.ns;
  const int rows = ns * j.group;  // row r = h * ns + k
  // Piece k of the sequence lies in chunk w_first + k: in that chunk's first slot, except piece 0
  // when the sequence begins inside its chunk (then it is the chunk's last piece, slot 1).
  const auto row_of = [&](int h, int k) -> int64_t {
    return (int64_t)(2 * (j.w_first + k) + (k == 0 ? j.which0 : 0)) * j.num_q_heads + j.hq0 + h;
  };
  // (h, k) of the row after (h, k); `on` false keeps it (the row after the last stays the last).
  // Written with selects, not branches: everything here is the same in all lanes, but the
  // compiler cannot know, and a branch with its reconvergence per row costs more than the maths.
  const auto advance = [&](int& h, int& k, bool on) {
    const int k2 = k + 1;
    const bool wrap = on & (k2 == ns);
    k = on ? (wrap ? 0 : k2) : k;
    h += wrap ? 1 : 0;
  };
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float big = -INFINITY, den = 0.f;
  int h_base = 0, k_base = 0;  // (h, k) of row r0
  for (int r0 = 0; r0 < rows; r0 += RB) {
    // All loads of a batch are unconditional (rows past the end repeat the last one) so that
    // they leave back to back: one round trip to L2 per batch.
    float4 xv[RB];
    float m_mine, l_mine;
    {
      const int r = min(r0 + lane, rows - 1);
      const int h = r / ns, k = r - h * ns;
      const int64_t row = row_of(h, k);
#ifdef PFD_BOUNDS_CHECK
      if (row < 0 || row >= j.ws_rows) { if (j.report) *j.report = (unsigned long long)row | (1ull << 63); return; }
#endif
      m_mine = __ldcg(j.pm + row);
      l_mine = __ldcg(j.pl + row);
      if (r0 + lane >= rows) { m_mine = -INFINITY; l_mine = 0.f; }  // no such row: weight 0 below
    }
    {
      int h = h_base, k = k_base;
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        xv[u] = __ldcg(reinterpret_cast<const float4*>(j.po + row_of(h, k) * D) + lane);
        advance(h, k, r0 + u + 1 < rows);
      }
    }
    // Scheduling fence: an empty statement that takes all 128 loaded values, so that no use of a
    // row can be moved in front of the load of a later row (which would serialise the loads).
    static_assert(RB == 32, "the statement below names 32 rows");
    asm volatile("" : "+f"(xv[0].x), "+f"(xv[0].y), "+f"(xv[0].z), "+f"(xv[0].w), "+f"(xv[1].x), "+f"(xv[1].y), "+f"(xv[1].z), "+f"(xv[1].w), "+f"(xv[2].x), "+f"(xv[2].y), "+f"(xv[2].z), "+f"(xv[2].w), "+f"(xv[3].x), "+f"(xv[3].y), "+f"(xv[3].z), "+f"(xv[3].w), "+f"(xv[4].x), "+f"(xv[4].y), "+f"(xv[4].z), "+f"(xv[4].w), "+f"(xv[5].x), "+f"(xv[5].y), "+f"(xv[5].z), "+f"(xv[5].w), "+f"(xv[6].x), "+f"(xv[6].y), "+f"(xv[6].z), "+f"(xv[6].w), "+f"(xv[7].x), "+f"(xv[7].y), "+f"(xv[7].z), "+f"(xv[7].w), "+f"(xv[8].x), "+f"(xv[8].y), "+f"(xv[8].z), "+f"(xv[8].w), "+f"(xv[9].x), "+f"(xv[9].y), "+f"(xv[9].z), "+f"(xv[9].w), "+f"(xv[10].x), "+f"(xv[10].y), "+f"(xv[10].z), "+f"(xv[10].w), "+f"(xv[11].x), "+f"(xv[11].y), "+f"(xv[11].z), "+f"(xv[11].w), "+f"(xv[12].x), "+f"(xv[12].y), "+f"(xv[12].z), "+f"(xv[12].w), "+f"(xv[13].x), "+f"(xv[13].y), "+f"(xv[13].z), "+f"(xv[13].w), "+f"(xv[14].x), "+f"(xv[14].y), "+f"(xv[14].z), "+f"(xv[14].w), "+f"(xv[15].x), "+f"(xv[15].y), "+f"(xv[15].z), "+f"(xv[15].w), "+f"(xv[16].x), "+f"(xv[16].y), "+f"(xv[16].z), "+f"(xv[16].w), "+f"(xv[17].x), "+f"(xv[17].y), "+f"(xv[17].z), "+f"(xv[17].w), "+f"(xv[18].x), "+f"(xv[18].y), "+f"(xv[18].z), "+f"(xv[18].w), "+f"(xv[19].x), "+f"(xv[19].y), "+f"(xv[19].z), "+f"(xv[19].w), "+f"(xv[20].x), "+f"(xv[20].y), "+f"(xv[20].z), "+f"(xv[20].w), "+f"(xv[21].x), "+f"(xv[21].y), "+f"(xv[21].z), "+f"(xv[21].w), "+f"(xv[22].x), "+f"(xv[22].y), "+f"(xv[22].z), "+f"(xv[22].w), "+f"(xv[23].x), "+f"(xv[23].y), "+f"(xv[23].z), "+f"(xv[23].w), "+f"(xv[24].x), "+f"(xv[24].y), "+f"(xv[24].z), "+f"(xv[24].w), "+f"(xv[25].x), "+f"(xv[25].y), "+f"(xv[25].z), "+f"(xv[25].w), "+f"(xv[26].x), "+f"(xv[26].y), "+f"(xv[26].z), "+f"(xv[26].w), "+f"(xv[27].x), "+f"(xv[27].y), "+f"(xv[27].z), "+f"(xv[27].w), "+f"(xv[28].x), "+f"(xv[28].y), "+f"(xv[28].z), "+f"(xv[28].w), "+f"(xv[29].x), "+f"(xv[29].y), "+f"(xv[29].z), "+f"(xv[29].w), "+f"(xv[30].x), "+f"(xv[30].y), "+f"(xv[30].z), "+f"(xv[30].w), "+f"(xv[31].x), "+f"(xv[31].y), "+f"(xv[31].z), "+f"(xv[31].w));
    int h = h_base, k = k_base;
#pragma unroll
    for (int u = 0; u < RB; ++u) {
      const bool live = r0 + u < rows;
      const float mv = __shfl_sync(0xffffffffu, m_mine, u);  // -inf for rows past the end
      const float lv = __shfl_sync(0xffffffffu, l_mine, u);
      const bool first = k == 0;
      const float big_in = first ? -INFINITY : big;
      const float m_new = fmaxf(big_in, mv);
      const float keep = (big_in == -INFINITY) ? 0.f : expf(big_in - m_new);
      const float c = (mv == -INFINITY) ? 0.f : expf(mv - m_new);
      den = den * keep + lv * c;
      acc[0] = acc[0] * keep + c * xv[u].x; acc[1] = acc[1] * keep + c * xv[u].y;
      acc[2] = acc[2] * keep + c * xv[u].z; acc[3] = acc[3] * keep + c * xv[u].w;
      big = m_new;
      const bool last = live & (k == ns - 1);
      const int hq = j.hq0 + h;
      if constexpr (PACKED) {
        float* dst = j.packed + ((int64_t)j.b * j.num_q_heads + hq) * (D + 2);
        if (last) {
          *reinterpret_cast<float2*>(dst + lane * 4) = make_float2(acc[0], acc[1]);
          *reinterpret_cast<float2*>(dst + lane * 4 + 2) = make_float2(acc[2], acc[3]);
          if (lane == 0) { dst[D] = big; dst[D + 1] = den; }
        }
      } else {
        const float inv = 1.f / den;
        uint16_t* dst = reinterpret_cast<uint16_t*>(j.output) + (int64_t)j.b * j.o_stride_b + (int64_t)hq * j.o_stride_h + lane * 4;
        uint32_t w0, w1;
        if constexpr (QBF16) {
          __nv_bfloat162 x = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
          __nv_bfloat162 y = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
          w0 = *reinterpret_cast<uint32_t*>(&x);
          w1 = *reinterpret_cast<uint32_t*>(&y);
        } else {
          w0 = pack_f16x2(acc[0] * inv, acc[1] * inv);
          w1 = pack_f16x2(acc[2] * inv, acc[3] * inv);
        }
        if (last) *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
      }
      advance(h, k, live);
    }
    h_base = h;
    k_base = k;
  }
}

// Rows of sequences with nothing to attend (seq_len <= kv_start): zeros, or (0, -inf, 0) packed.
// The merge kernel writes them when it runs; with a plan the chunk kernel does, sequence b by
// warp b mod (warps of the grid).
template <int D>
__device__ __forceinline__ void write_empty_sequence(const KernelParams& p, int b, int lane) {
  for (int hq = 0; hq < p.num_q_heads; ++hq) {
    if (p.packed_output != nullptr) {
      float* dst = p.packed_output + ((int64_t)b * p.num_q_heads + hq) * (D + 2);
      for (int d = lane; d < D; d += 32) dst[d] = 0.f;
      if (lane == 0) { dst[D] = -INFINITY; dst[D + 1] = 0.f; }
    } else {
      uint16_t* dst = reinterpret_cast<uint16_t*>(p.output) + (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h;
      for (int d = lane; d < D; d += 32) dst[d] = 0;
    }
  }
}

// grid = one CTA per SM; block = NWARPS independent warps.  KV16 = false: e4m3 caches;
// true: caches in the query's 16-bit type (the reference's non-quantised sibling operator).
// cp.plan == nullptr: every CTA derives the work split itself; with a plan it is read.  The
// merge kernel behind combines the pieces of cut sequences -- unless FUSED (needs a plan): then
// the warp whose piece of a sequence arrives last combines them in here and no merge kernel
// follows.  FUSED is a separate instantiation because the merge code costs the streaming loop
// registers; on B200 it is the slower of the two (one warp per sequence and kv head merges
// where the merge kernel has a warp per row).
template <bool QBF16, int NSTAGE, int NWARPS, bool KV16 = false, bool FUSED = false>
__global__ void __launch_bounds__(NWARPS * 32, 1)
paged_decode_fp8_chunk_kernel(const KernelParams p, const TmaParams tp, const ChunkParams cp,
                              const __grid_constant__ CUtensorMap tmap_k,
                              const __grid_constant__ CUtensorMap tmap_v) {
  constexpr int D = 128;
  constexpr int NT = NWARPS * 32;
  constexpr uint32_t kTile = (KV16 ? 2 : 1) * kPage * D;
  constexpr uint32_t kStage = 4 * kTile;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_v)) : "memory");
  }
  // A programmatic dependent of whatever precedes it in the stream (normally the previous
  // layer-step's last kernel, which may still read the workspace): no memory access before that
  // kernel has completed -- except, if the caller vouches that the preceding kernel does not
  // write them, the reads of seq_lens, block_table and the plan.
  if (!p.early_metadata) pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, i = lane >> 2, j = lane & 3;
  const int B = cp.batch, hkv = p.num_kv_heads;
  const int page_first = p.kv_start / kPage;
  const int W = (int)blockIdx.x * NWARPS + warp;
  const int grp = W / hkv, kvh = W - grp * hkv;  // one warp per kv head and group
  const int num_groups = cp.num_warps / hkv;
  const bool planned = cp.plan != nullptr;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t bars = ring + NWARPS * NSTAGE * kStage;
  int32_t* sm_scan = reinterpret_cast<int32_t*>(base + NWARPS * NSTAGE * kStage + NWARPS * NSTAGE * 8);  // [NWARPS]
  int32_t* prefix = sm_scan + NWARPS;  // [B + 1] pairs before sequence b
  int32_t* lens = prefix + (B + 1);    // [B]
  const PairList list{prefix, lens, B, page_first, p.kv_start};

  mark_phase_at(tp, W, 0, lane == 0);  // start
  mark_value_at(tp, W, 5, lane == 0, sm_id());
  const uint32_t my_ring = ring + warp * NSTAGE * kStage;
  const uint32_t my_bars = bars + warp * NSTAGE * 8;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) mbar_init(my_bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies' completions see initialised barriers
  }

  int total;
  ChunkRange cr;
  int32_t ids_cur;
  uint32_t seq_ends = 0xffffffffu;  // of the first pairs, those that hold a sequence's last page
  bool plan_ok = true;
  if (planned) {
    // one round trip: header, this group's range and the page ids of its first 16 pairs.  Every
    // lane reads the same header words (broadcast loads), so nothing below depends on the lane.
    const int32_t* gw = cp.plan + plan_groups_off(B) + (int64_t)min(grp, num_groups - 1) * kPlanGroupWords;
    const int4 h0 = __ldg(reinterpret_cast<const int4*>(cp.plan));      // magic, batch, kv_start, kv heads
    const int4 h1 = __ldg(reinterpret_cast<const int4*>(cp.plan) + 1);  // groups, piece cost, total, indptr
    const int4 g0 = __ldg(reinterpret_cast<const int4*>(gw));  // P0, P1, pairs that end a sequence
    cr.P0 = g0.x;
    cr.P1 = g0.y;
    seq_ends = (uint32_t)g0.z;
    ids_cur = __ldg(gw + 4 + lane);
    plan_ok = h0.x == kPlanMagic && h0.y == B && h0.z == p.kv_start && h0.w == hkv && h1.x == num_groups &&
              h1.y == cp.piece_cost && h1.w == (p.page_indptr != nullptr ? 1 : 0);
    total = h1.z;
    if (grp >= num_groups || !plan_ok) { cr.P0 = cr.P1 = total; ids_cur = -1; }
    // prefix sum and lengths into shared memory; used only after the barrier further down
    for (int x = threadIdx.x; x < 2 * B + 1; x += NT) prefix[x] = __ldg(cp.plan + kPlanHeaderWords + x);
  } else {
    scan_pairs<NT>(p.seq_lens, B, p.kv_start, sm_scan, prefix, lens);  // ends with the last CTA-wide barrier
    total = prefix[B];
  }
  mark_phase_at(tp, W, 1, lane == 0);  // split known
  const Chunking chunks(total, B, max(num_groups, 1), cp.piece_cost);
  const int C0 = chunks.start_of(grp);
  if (!planned) {
    cr = chunk_range(list, chunks, grp);
    ids_cur = fetch_ids(list, p, cr, 0, lane);
  }
  const int P0 = cr.P0, P1 = cr.P1;
  const int n = P1 - P0;

  auto fire = [&](int t, int32_t ids, int base_t) {  // all lanes call; lane 0 issues
    const int32_t phys0 = __shfl_sync(0xffffffffu, ids, (2 * (t - base_t)) & 31);
    const int32_t phys1 = __shfl_sync(0xffffffffu, ids, (2 * (t - base_t) + 1) & 31);
    if (lane == 0) {
      const uint32_t bar = my_bars + 8 * (t % NSTAGE);
      const uint32_t dst = my_ring + (t % NSTAGE) * kStage;
      const bool two = phys1 >= 0;
      mbar_expect_tx(bar, two ? kStage : kStage / 2);
      const int c1 = tp.head_is_dim1 ? kvh : 0;
      const int c2 = tp.head_is_dim1 ? 0 : kvh;
      const uint64_t pol = l2_policy_evict_first();
      const auto load = [&](uint32_t to, const CUtensorMap* map, int32_t phys) {
        if constexpr (KV16) {  // two halves of 64 elements
          if (p.kv_evict_first) {
            tma_load_tile_x(to, map, bar, 0, c1, c2, phys, pol);
            tma_load_tile_x(to + kTile / 2, map, bar, 64, c1, c2, phys, pol);
          } else {
            tma_load_tile_x(to, map, bar, 0, c1, c2, phys);
            tma_load_tile_x(to + kTile / 2, map, bar, 64, c1, c2, phys);
          }
        } else {
          if (p.kv_evict_first) tma_load_tile(to, map, bar, c1, c2, phys, pol);
          else tma_load_tile(to, map, bar, c1, c2, phys);
        }
      };
      load(dst, &tmap_k, phys0);
      load(dst + 2 * kTile, &tmap_v, phys0);
      if (two) {
        load(dst + kTile, &tmap_k, phys1);
        load(dst + 3 * kTile, &tmap_v, phys1);
      }
    }
  };
  __syncwarp();
  // early_kv: the preceding kernel writes K/V only into each sequence's last page, so the first
  // copies go out before it has completed -- except pairs that hold such a page
  const bool early_kv = planned && p.early_metadata && p.early_kv && plan_ok;
  if (early_kv) {
#pragma unroll
    for (int t = 0; t < NSTAGE; ++t)
      if (t < n && !((seq_ends >> t) & 1u)) fire(t, ids_cur, 0);
  }
  if (p.early_metadata) pdl_wait();
  const uint32_t xstep = exchange_step(p);  // behind the wait: the previous step's merge advances it
#pragma unroll
  for (int t = 0; t < NSTAGE; ++t)
    if (t < n && (!early_kv || ((seq_ends >> t) & 1u))) fire(t, ids_cur, 0);
  mark_phase_at(tp, W, 2, lane == 0);  // first copies issued
  if (planned) {
    __syncthreads();  // the last CTA-wide barrier: prefix and lens are in shared memory
    if (!plan_ok) {   // a plan made for another call: nothing is computed, the host reads the status word
      if (threadIdx.x == 0) atomicExch(tp.status, kErrPlanMismatch);
      return;
    }
    if constexpr (FUSED)  // rows of sequences with nothing to attend
      for (int b = W; b < B; b += cp.num_warps)
        if (prefix[b + 1] == prefix[b]) write_empty_sequence<D>(p, b, lane);
  }
  if (n <= 0) return;  // (any pdl_wait this grid owes has been executed above)

  int32_t ids_next = fetch_ids(list, p, cr, 16, lane);
  int ids_base = 0;

  // swizzled shared-memory offsets of this thread's fragments inside a tile
  uint32_t k_off[2][2], v_off[4];
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int l = 0; l < 2; ++l)
      k_off[half][l] = (half * 8 + rho(i)) * D + (((j + 4 * l) ^ rho(i)) << 4);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = v_row(j, r);
    v_off[r] = row * D + ((i ^ (row & 7)) << 4);
  }

  // ---- consumer side: the pieces of the chunk in order
  struct Cursor { int b, np, start; };  // current sequence, its pairs, list index of its first pair
  Cursor cur;
  cur.b = list.seq_of(P0);
  cur.np = prefix[cur.b + 1] - prefix[cur.b];
  cur.start = prefix[cur.b];
  const float ks = KV16 ? 1.f : (p.k_scale_ph ? __ldg(p.k_scale_ph + kvh) : p.k_scale);
  const float vs = KV16 ? 1.f : (p.v_scale_ph ? __ldg(p.v_scale_ph + kvh) : p.v_scale);
  const float scale_log2 = ks * p.sm_scale * kLog2e;
  const auto load_q = [&](uint32_t (&dst)[1][8][2], int b) {
    if constexpr (KV16) kv16_load_q(dst, p, b, kvh, i, j);
    else bal_load_q<QBF16, 1>(dst, p, b, kvh, i, j);
  };
  uint32_t qb[1][8][2];
  load_q(qb, cur.b);
  BalState<1> st;
  bool ok = true;
  int t = 0;  // pairs consumed
  int g = P0;
#pragma unroll 1
  while (ok && g < P1) {
    const int e = min(cur.start + cur.np, P1);
    const int piece_first = g;
    // the next piece's query is requested now and used when this piece is done
    Cursor nxt = cur;
    uint32_t qn[1][8][2];
    if (e < P1) {
      do {  // sequences with nothing to attend have no pairs
        nxt.start += nxt.np;
        ++nxt.b;
        nxt.np = prefix[nxt.b + 1] - prefix[nxt.b];
      } while (nxt.np == 0);
      load_q(qn, nxt.b);
    }
    const int seq_len = lens[cur.b];
    const bool whole = cur.start >= P0 && cur.start + cur.np <= P1;
    bal_reset<1>(st);
#pragma unroll 1
    for (; g < e; ++g, ++t) {
      const int s = t % NSTAGE;
      if (!mbar_wait_bounded(my_bars + 8 * s, (t / NSTAGE) & 1, tp.wait_limit_ns)) { ok = false; break; }
      if (t == 0) mark_phase_at(tp, W, 3, lane == 0);  // first data landed
      if (t == n / 2) mark_phase_at(tp, W, 6, lane == 0);  // half of the chunk consumed
      const int tok0 = (page_first + 2 * (g - cur.start)) * kPage;
      if constexpr (KV16) kv16_step<QBF16>(st, my_ring + s * kStage, qb, scale_log2, tok0, p.kv_start, seq_len, lane);
      else bal_step<1>(st, my_ring + s * kStage, k_off, v_off, qb, scale_log2, tok0, p.kv_start, seq_len, i, j);
      // all reads of the stage fed MMAs above: hand it back to TMA for the chunk's pair t + NSTAGE
      __syncwarp();
      const int tn = t + NSTAGE;
      if (tn < n) {
        if ((tn & 15) == 0) {
          ids_cur = ids_next;
          ids_base = tn;
          ids_next = fetch_ids(list, p, cr, tn + 16, lane);
        }
        if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        fire(tn, ids_cur, ids_base);
      }
    }
    if (!ok) break;

    // ---- the piece is complete: this thread's sums over the tokens it saw
    float lsum[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float x = st.l[0][c];
      x += __shfl_xor_sync(0xffffffffu, x, 4);
      x += __shfl_xor_sync(0xffffffffu, x, 8);
      x += __shfl_xor_sync(0xffffffffu, x, 16);
      lsum[c] = x;
    }
    const int s0 = chunks.first_unit(cur.start, cur.b);
    const int which = s0 > C0 ? 1 : 0;
#ifdef PFD_BOUNDS_CHECK
    if (!whole && chunk_slot_row(grp, which, p.num_q_heads, p.num_q_heads - 1) >= p.dbg_ws_rows)
      mark_value_at(tp, 2 * cp.num_warps + 2, 0, lane == 0, ((unsigned long long)(unsigned)grp << 32) | (unsigned)which);
    if (cur.b < 0 || cur.b >= B) mark_value_at(tp, 2 * cp.num_warps + 4, 0, lane == 0, (unsigned long long)(unsigned)cur.b);
#endif
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int row = 2 * j + c;
      if (row >= p.group) continue;
      const int hq = kvh * p.group + row;
      if constexpr (KV16) {
        // natural layout: this thread holds d = 16 mt + i and 16 mt + i + 8 of the row
        const float m_nat = st.m[0][c] * kLn2;
        const int64_t r = whole ? 0 : chunk_slot_row(grp, which, p.num_q_heads, hq);
        const float inv = 1.f / lsum[c];
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int d = 16 * mt + i + 8 * hh;
            const float x = st.o[0][mt][2 * hh + c];
            if (!whole) {
              store_partial_scalar(p.partial_output, p.partial_dtype, r * D + d, x);
            } else if (p.packed_output != nullptr) {
              p.packed_output[((int64_t)cur.b * p.num_q_heads + hq) * (D + 2) + d] = x;
            } else {
              const int64_t o = (int64_t)cur.b * p.o_stride_b + (int64_t)hq * p.o_stride_h + d;
              if constexpr (QBF16) reinterpret_cast<__nv_bfloat16*>(p.output)[o] = __float2bfloat16_rn(x * inv);
              else reinterpret_cast<__half*>(p.output)[o] = __float2half_rn(x * inv);
            }
          }
        if (i == 0) {
          if (!whole) {
            p.partial_max[r] = m_nat;
            p.partial_sum[r] = lsum[c];
          } else if (p.packed_output != nullptr) {
            float* dst = p.packed_output + ((int64_t)cur.b * p.num_q_heads + hq) * (D + 2);
            dst[D] = m_nat;
            dst[D + 1] = lsum[c];
          }
        }
      } else {
        float v[16];
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          v[2 * mt] = st.o[0][mt][c] * vs;
          v[2 * mt + 1] = st.o[0][mt][2 + c] * vs;
        }
        if (whole) {
          store_row16<QBF16>(p, cur.b, hq, 16 * i, v, st.m[0][c] * kLn2, lsum[c], i == 0, xstep);
        } else {
          const int64_t r = chunk_slot_row(grp, which, p.num_q_heads, hq);
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.partial_output) + r * D + 16 * i);
#pragma unroll
          for (int f = 0; f < 4; ++f) dst[f] = make_float4(v[4 * f], v[4 * f + 1], v[4 * f + 2], v[4 * f + 3]);
          if (i == 0) {
            p.partial_max[r] = st.m[0][c] * kLn2;
            p.partial_sum[r] = lsum[c];
          }
        }
      }
    }
    if constexpr (FUSED) if (!whole) {
      // Publish the piece, then count this warp's pairs of the sequence in: the warp that
      // completes the count finds every other piece in L2 and writes the final rows.
      __threadfence();
      __syncwarp();
      const int mine = e - piece_first;
      int32_t* counter = cp.plan + plan_counters_off(B, num_groups) + (int64_t)cur.b * hkv + kvh;
#ifdef PFD_BOUNDS_CHECK
      if (cur.b < 0 || cur.b >= B || mine <= 0 || mine > cur.np) {
        mark_value_at(tp, 2 * cp.num_warps + 3, 0, lane == 0, ((unsigned long long)(unsigned)cur.b << 32) | (unsigned)mine);
        mark_value_at(tp, 2 * cp.num_warps + 3, 1, lane == 0, ((unsigned long long)(unsigned)cur.np << 32) | (unsigned)W);
      }
#endif
      int before = 0;
      if (lane == 0) before = atomicAdd(counter, mine);
      before = __shfl_sync(0xffffffffu, before, 0);
      if (before + mine == cur.np) {
        __threadfence();
        mark_phase_at(tp, cp.num_warps + W, 0, lane == 0);  // merge begins
        MergeJob job;
        job.po = reinterpret_cast<const float*>(p.partial_output);
        job.pm = p.partial_max;
        job.pl = p.partial_sum;
        job.output = p.output;
        job.packed = p.packed_output;
        job.o_stride_b = p.o_stride_b;
        job.o_stride_h = p.o_stride_h;
        job.num_q_heads = p.num_q_heads;
        job.hq0 = kvh * p.group;
        job.group = p.group;
        job.w_first = chunks.chunk_of(s0);
        job.ns = chunks.chunk_of(s0 + 2 * (cur.np - 1)) - job.w_first + 1;
        job.which0 = s0 > chunks.start_of(job.w_first) ? 1 : 0;
        job.b = cur.b;
#ifdef PFD_BOUNDS_CHECK
        job.ws_rows = p.dbg_ws_rows;
        job.report = tp.phase_times ? tp.phase_times + (size_t)(2 * cp.num_warps + 1) * 8 : nullptr;
#endif
        if (p.packed_output != nullptr) merge_pieces_of_sequence<QBF16, true>(job, lane);
        else merge_pieces_of_sequence<QBF16, false>(job, lane);
        if (lane == 0) *counter = 0;  // ready for the next launch that uses this plan
        mark_phase_at(tp, cp.num_warps + W, 1, lane == 0);  // merged
      }
    }
    cur = nxt;
#pragma unroll
    for (int f = 0; f < 8; ++f) { qb[0][f][0] = qn[0][f][0]; qb[0][f][1] = qn[0][f][1]; }
  }
  mark_phase_at(tp, W, 4, lane == 0);  // chunk done
  mark_value_at(tp, W, 7, lane == 0, (unsigned long long)n);
  if (!ok && lane == 0) {
    // a copy never landed: record it; give the copies still in flight a bounded chance to land
    atomicExch(tp.status, kErrTmaTimeout);
    const int issued = min(n, t + NSTAGE);
    for (int u = t + 1; u < issued; ++u) mbar_wait_bounded(my_bars + 8 * (u % NSTAGE), (u / NSTAGE) & 1, tp.wait_limit_ns);
  }
}

// LSE merge of the pieces the chunk kernel left in the workspace.  WPR = 1: one warp per
// (sequence, q head) row, four rows per CTA; WPR = 4: the four warps of a CTA share one row,
// warp w taking pieces w, w + 4, ..., and combine through shared memory.  KB pieces are
// requested per round trip (rows with at most four pieces take a shorter code path); MINB is
// the CTAs per SM the register budget is held to.  A row whose sequence lay inside one chunk
// has been written already.  Same maths as _paged_split_kv_reduce
// (integrations/vllm/l20_paged_split_kv.py:459-488).
template <bool QBF16, int WPR, int KB, int MINB>
__global__ void __launch_bounds__(128, MINB)
paged_decode_chunk_merge_kernel(const KernelParams p, const TmaParams tp, const ChunkParams cp) {
  constexpr int D = 128, E = 4;
  static_assert(WPR == 1 || WPR == 4, "one or four warps per row");
  pdl_launch_dependents();
  mark_phase_at(tp, cp.num_warps + blockIdx.x, 5, threadIdx.x == 0);  // merge CTA resident
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = WPR == 1 ? blockIdx.x * (blockDim.x >> 5) + warp : blockIdx.x;  // WPR == 1: one row per warp of the CTA
  const int part = WPR == 1 ? 0 : warp;
  // This grid must not complete before the chunk kernel has (the next kernel of the stream would
  // start while the chunk kernel is still writing): CTAs with nothing to do leave at once, which
  // frees their slots for the rows that have, but the last CTA of the grid always waits.
  const bool keeper = blockIdx.x == gridDim.x - 1;
  if (row >= cp.batch * p.num_q_heads) {  // WPR == 1 only: whole warps, no barrier below
    if (keeper) pdl_wait();
    return;
  }
  const int b = row / p.num_q_heads, hq = row % p.num_q_heads;
  // seq_lens is an input of the whole step, not a result of the chunk kernel: the chunking is
  // read from the plan, or recomputed here, while that kernel is still running.
  int below = 0, all = 0, np = 0;
  if (cp.plan != nullptr) {
    const int32_t* pre = cp.plan + kPlanHeaderWords;
    below = __ldg(pre + b);
    np = __ldg(pre + b + 1) - below;
    all = __ldg(pre + cp.batch);
  } else {
    for (int x = lane; x < cp.batch; x += 32) {
      const int n = pairs_of(__ldg(p.seq_lens + x), p.kv_start);
      all += n;
      below += x < b ? n : 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      all += __shfl_xor_sync(0xffffffffu, all, off);
      below += __shfl_xor_sync(0xffffffffu, below, off);
    }
    np = pairs_of(__ldg(p.seq_lens + b), p.kv_start);
  }
  const Chunking chunks(all, cp.batch, max(cp.num_warps / p.num_kv_heads, 1), cp.piece_cost);
  const int s0 = chunks.first_unit(below, b);
  const int w_first = np > 0 ? chunks.chunk_of(s0) : 0;
  const int ns = np > 0 ? chunks.chunk_of(s0 + 2 * (np - 1)) - w_first + 1 : 0;
  if (ns == 1) {  // written by the chunk kernel (the whole CTA returns: one row per CTA if WPR == 4)
    if (keeper) pdl_wait();
    return;
  }
  float acc[E] = {0.f, 0.f, 0.f, 0.f};
  float big = -INFINITY, den = 0.f;
  // pieces k0, k0 + WPR, ... (K of them) in one round trip, folded into (acc, big, den)
  auto round = [&](auto kc, int k0) {
    constexpr int K = decltype(kc)::value;
    float mv[K], lv[K];
    float4 xv[K];
#pragma unroll
    for (int u = 0; u < K; ++u) {
      const int k = k0 + u * WPR;
      const bool on = k < ns;
      const int w = w_first + (on ? k : 0);
      const int64_t r = chunk_slot_row(w, s0 > chunks.start_of(w) ? 1 : 0, p.num_q_heads, hq);
      mv[u] = on ? p.partial_max[r] : -INFINITY;
      lv[u] = on ? p.partial_sum[r] : 0.f;
      if (p.partial_dtype == 0) {
        xv[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.partial_output) + r * D + lane * E);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.partial_output) + r * D + lane * E);
        if (p.partial_dtype == 1) {
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
          const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
          xv[u] = make_float4(a.x, a.y, c.x, c.y);
        } else {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          xv[u] = make_float4(a.x, a.y, c.x, c.y);
        }
      }
    }
    float m_new = big;
#pragma unroll
    for (int u = 0; u < K; ++u) m_new = fmaxf(m_new, mv[u]);
    const float keep = (big == -INFINITY) ? 0.f : expf(big - m_new);
    den *= keep;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] *= keep;
#pragma unroll
    for (int u = 0; u < K; ++u) {
      const float c = (mv[u] == -INFINITY) ? 0.f : expf(mv[u] - m_new);
      den += lv[u] * c;
      acc[0] += c * xv[u].x; acc[1] += c * xv[u].y; acc[2] += c * xv[u].z; acc[3] += c * xv[u].w;
    }
    big = m_new;
  };
  pdl_wait();  // the chunk kernel's stores are complete and visible from here on
  const uint32_t xstep = exchange_step(p);  // issued here, needed only when the row is stored
  mark_phase_at(tp, cp.num_warps + blockIdx.x, 6, threadIdx.x == 0);  // chunk kernel complete
  if (WPR == 1 && ns <= 4) {
    if (ns > 0) round(std::integral_constant<int, 4>{}, 0);
  } else {
    for (int k0 = part; k0 < ns; k0 += KB * WPR) round(std::integral_constant<int, KB>{}, k0);
  }
  if constexpr (WPR == 4) {
    // combine the four warps' (acc, big, den) of this row; warp 0 finishes
    __shared__ __align__(16) float sh_acc[4][D];
    __shared__ float sh_m[4], sh_l[4];
    *reinterpret_cast<float4*>(&sh_acc[warp][lane * E]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (lane == 0) { sh_m[warp] = big; sh_l[warp] = den; }
    __syncthreads();
    if (warp != 0) return;
    float m_all = fmaxf(fmaxf(sh_m[0], sh_m[1]), fmaxf(sh_m[2], sh_m[3]));
    den = 0.f;
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (sh_m[w] == -INFINITY) ? 0.f : expf(sh_m[w] - m_all);
      const float4 x = *reinterpret_cast<const float4*>(&sh_acc[w][lane * E]);
      den += sh_l[w] * c;
      acc[0] += c * x.x; acc[1] += c * x.y; acc[2] += c * x.z; acc[3] += c * x.w;
    }
    big = m_all;
  }
  if (p.xch_world > 0) {
    for (int dest = 0; dest < p.xch_world; ++dest) {
      unsigned long long* dst = xch_row(p, dest, row, xstep);
      xch_store2(dst + lane * E, acc[0], acc[1], xstep);
      xch_store2(dst + lane * E + 2, acc[2], acc[3], xstep);
      if (lane == 0) xch_store2(dst + D, big, den, xstep);
    }
    mark_phase_at(tp, cp.num_warps + blockIdx.x, 7, threadIdx.x == 0);  // merged and sent
    return;
  }
  if (p.packed_output != nullptr) {
    float* dst = p.packed_output + (int64_t)row * (D + 2);
    *reinterpret_cast<float2*>(dst + lane * E) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2*>(dst + lane * E + 2) = make_float2(acc[2], acc[3]);
    if (lane == 0) { dst[D] = big; dst[D + 1] = den; }
    return;
  }
  mark_phase_at(tp, cp.num_warps + blockIdx.x, 7, threadIdx.x == 0);  // merged
  const float inv = ns > 0 ? 1.f / den : 0.f;
  uint16_t* dst = reinterpret_cast<uint16_t*>(p.output) + (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h + lane * E;
  uint32_t w0, w1;
  if constexpr (QBF16) {
    __nv_bfloat162 x = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
    __nv_bfloat162 y = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
    w0 = *reinterpret_cast<uint32_t*>(&x);
    w1 = *reinterpret_cast<uint32_t*>(&y);
  } else {
    w0 = pack_f16x2(acc[0] * inv, acc[1] * inv);
    w1 = pack_f16x2(acc[2] * inv, acc[3] * inv);
  }
  *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
}

}  // namespace pfd
