// Balanced, persistent form of the split-KV decode step for head_dim 128 (sm_100a).
//
// Instead of a grid of fixed (sequence, kv head, split) work items, a fixed number of CTAs
// (a multiple of the SM count) share the flattened list of page pairs of all (sequence,
// kv head) segments in equal contiguous chunks, so every CTA streams the same number of KV
// bytes whatever the mix of context lengths.  A CTA walks the segments its chunk overlaps;
// its four compute warps take the chunk's page pairs round-robin, each through a private TMA
// ring that keeps loading across segment boundaries, and reduce their (m, l, O) for a segment
// in shared memory.  A fifth warp retires segments: it turns the reduced sums into the final
// output, or -- for a segment that straddles chunks -- into an (o, m, l) piece in the caller's
// workspace, and the CTA that retires the last piece (a per-segment semaphore) merges them.
// The compute warps never wait for a global-memory round trip at a segment boundary, and
// there is no second kernel launch.  Whole segments of at most kSoloPairs page pairs skip the
// CTA-level reduction altogether: one warp streams them and writes their output itself.
//
// Maths per page pair and warp, "heads as columns": S^T = K Q^T and O^T += V^T P^T with
// mma.sync.m16n8k16 (f16 in, f32 accumulate).  Tokens (resp. head-dim rows) fill the 16-row M
// dimension and the <= 8 query heads of the group fill N = 8 exactly, so nothing of the tile is
// padding, O^T needs 32 accumulator registers, and P^T reaches its B-fragment layout with one
// movmatrix per 8 tokens.
#pragma once

#include "paged_decode_kernels.cuh"

namespace pfd {

struct BalancedParams {
  int32_t batch;
  int32_t min_chunk;        // lower bound on pairs per CTA so that pieces fit the workspace
  int32_t workspace_splits; // capacity of the workspace's split axis
  int32_t* semaphores;      // [batch * num_kv_heads], zero between calls
};

constexpr int kErrWorkspace = 2;

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

// Segment cursor over the flattened pair list (uniform across a warp).
struct SegCursor {
  int b, kvh;  // current segment
  int np;      // page pairs in it
  int start;   // global pair index of its first pair
};

// Advance `c` until its segment contains global pair `gp` (gp < total is the caller's duty).
__device__ __forceinline__ void seg_seek(SegCursor& c, int gp, const int32_t* prefix, int hkv) {
  while (gp >= c.start + c.np) {
    c.start += c.np;
    if (++c.kvh == hkv) {
      c.kvh = 0;
      ++c.b;
      c.np = prefix[c.b + 1] - prefix[c.b];
    }
  }
}

// The part of one segment that lies inside a CTA's chunk [P0, P1).
struct Piece {
  int b, kvh;
  int seg_start, np;  // the whole segment
  int a, e;           // global pair range of the piece
  int owner;          // >= 0: a small whole segment handled by that compute warp alone ("solo")
  __device__ __forceinline__ bool solo() const { return owner >= 0; }
};

constexpr int kSoloPairsMin = 4;
constexpr int kComputeWarps = 4;
constexpr int kBarMax = 1, kBarReady = 2, kBarFree = 3;  // named barriers (0 is __syncthreads)

// Walks the pieces of a chunk in order.  Every walker (each compute warp's producer and
// consumer side, and the retiring warp) sees the same pieces with the same owners: a solo piece
// goes to the compute warp with the least work assigned so far.
struct PieceWalker {
  SegCursor c;
  int P0, P1, solo_max;
  int load[kComputeWarps];  // pairs assigned to each compute warp so far

  __device__ __forceinline__ void init(const SegCursor& first, int p0, int p1, int chunk) {
    c = first; P0 = p0; P1 = p1;
    solo_max = max(kSoloPairsMin, chunk >> 3);
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w) load[w] = 0;
  }
  // The piece that contains global pair g (P0 <= g < P1); call with increasing g only.
  __device__ __forceinline__ Piece at(int g, const int32_t* prefix, int hkv) {
    seg_seek(c, g, prefix, hkv);
    Piece q;
    q.b = c.b; q.kvh = c.kvh; q.seg_start = c.start; q.np = c.np;
    q.a = max(c.start, P0);
    q.e = min(c.start + c.np, P1);
    q.owner = -1;
    const int len = q.e - q.a;
    if (q.a == c.start && q.e == c.start + c.np && c.np <= solo_max) {
      int best = 0, least = load[0];
#pragma unroll
      for (int w = 1; w < kComputeWarps; ++w)
        if (load[w] < least) { least = load[w]; best = w; }
      q.owner = best;
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w)
        if (w == best) load[w] += len;
    } else {
#pragma unroll
      for (int w = 0; w < kComputeWarps; ++w) load[w] += (len - w + kComputeWarps - 1) / kComputeWarps;
    }
    return q;
  }
};

// First pair of compute warp `warp` in piece `q` (>= q.e if it has none) and its stride.
__device__ __forceinline__ int piece_first(const Piece& q, int warp) {
  if (q.solo()) return q.owner == warp ? q.a : q.e;
  return q.a + warp;
}
__device__ __forceinline__ int piece_stride(const Piece& q) { return q.solo() ? 1 : kComputeWarps; }

__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// The accumulation buffer is [rows][32 float4]; float4 f of row `row` lives at f ^ ((row & 7) >> 1),
// which makes the compute warps' float4 read-modify-writes bank-conflict free.
__device__ __forceinline__ int acc_f4(int row, int f) { return row * 32 + (f ^ ((row & 7) >> 1)); }

template <bool QBF16>
__device__ __forceinline__ void store_row16(const KernelParams& p, int b, int hq, int d0, const float (&v)[16],
                                            float m_nat, float l, bool write_ml) {
  // 16 consecutive head-dim values of one (sequence, q head) row: final output or packed form
  if (p.packed_output != nullptr) {
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

// grid = persistent CTAs (a multiple of the SM count); block = 4 compute warps + 1 retiring warp.
template <bool QBF16, int NH, int NSTAGE>
__global__ void __launch_bounds__(160, (NH == 1 ? 3 : 1))
paged_decode_fp8_balanced_kernel(const KernelParams p, const TmaParams tp, const BalancedParams bp,
                                 const __grid_constant__ CUtensorMap tmap_k,
                                 const __grid_constant__ CUtensorMap tmap_v) {
  constexpr int D = 128;
  constexpr int NC = kComputeWarps;
  constexpr int NT = (NC + 1) * 32;
  constexpr uint32_t kTile = kPage * D;
  constexpr uint32_t kStage = 4 * kTile;
  constexpr int ROWS = 8 * NH;  // head rows of the accumulation buffer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, i = lane >> 2, j = lane & 3;
  const int B = bp.batch, hkv = p.num_kv_heads;
  const int page_first = p.kv_start / kPage;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base = smem_raw + (ring - smem_u32(smem_raw));
  uint8_t* after = base + NC * NSTAGE * kStage;
  const uint32_t bars = ring + NC * NSTAGE * kStage;
  float* sm_acc = reinterpret_cast<float*>(after + NC * NSTAGE * 8);  // [ROWS][D], swizzled, zero when free
  float* sm_m = sm_acc + ROWS * D;                                   // [NC][ROWS]
  float* sm_l = sm_m + NC * ROWS;                                    // [NC][ROWS]
  int32_t* sm_misc = reinterpret_cast<int32_t*>(sm_l + NC * ROWS);   // [1 .. NC+1] scan scratch
  int32_t* prefix = sm_misc + 8 + NC;                                // [B + 1] pairs before sequence b
  int32_t* lens = prefix + (B + 1);                                  // [B]

  mark_phase(tp, 0);  // start
  const uint32_t my_ring = ring + warp * NSTAGE * kStage;  // compute warps only
  const uint32_t my_bars = bars + warp * NSTAGE * 8;
  if (warp < NC && lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) mbar_init(my_bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int e = threadIdx.x; e < ROWS * D / 4; e += NT) reinterpret_cast<float4*>(sm_acc)[e] = make_float4(0.f, 0.f, 0.f, 0.f);

  // ---- pairs per sequence and their exclusive prefix sum (every CTA computes the same)
  {
    const int per = (B + NT - 1) / NT;
    const int b0 = threadIdx.x * per;
    int local = 0;
    for (int q = 0; q < per; ++q) {
      const int b = b0 + q;
      if (b < B) {
        const int len = p.seq_lens[b];
        lens[b] = len;
        const int pages = len > page_first * kPage ? (len + kPage - 1) / kPage - page_first : 0;
        local += (pages + 1) >> 1;
      }
    }
    int incl = local;  // inclusive scan over the CTA's threads
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += x;
    }
    if (lane == 31) sm_misc[1 + warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += sm_misc[1 + w];
    int run = before + incl - local;
    for (int q = 0; q < per; ++q) {
      const int b = b0 + q;
      if (b < B) {
        prefix[b] = run;
        const int len = lens[b];
        const int pages = len > page_first * kPage ? (len + kPage - 1) / kPage - page_first : 0;
        run += (pages + 1) >> 1;
      }
    }
    if (threadIdx.x == NT - 1) prefix[B] = before + incl;
    __syncthreads();
  }
  // Sequences with nothing to attend (seq_len <= kv_start) belong to no chunk: their rows are
  // filled here, zeros or (0, -inf, 0) in packed form, spread over all CTAs.
  for (int row = blockIdx.x * NT + threadIdx.x; row < B * p.num_q_heads; row += gridDim.x * NT) {
    const int b = row / p.num_q_heads, hq = row % p.num_q_heads;
    if (lens[b] > p.kv_start) continue;
    if (p.packed_output != nullptr) {
      float* dst = p.packed_output + (int64_t)row * (D + 2);
      for (int d = 0; d < D; ++d) dst[d] = 0.f;
      dst[D] = -INFINITY;
      dst[D + 1] = 0.f;
    } else {
      uint16_t* dst = reinterpret_cast<uint16_t*>(p.output) + (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h;
      for (int d = 0; d < D; ++d) dst[d] = 0;
    }
  }
  mark_phase(tp, 1);  // scan done
  const int total = prefix[B] * hkv;
  int chunk = (total + (int)gridDim.x - 1) / (int)gridDim.x;
  chunk = max(chunk, bp.min_chunk);
  const int P0 = min((int)blockIdx.x * chunk, total);
  const int P1 = min(P0 + chunk, total);
  if (P0 >= P1) return;

  // ---- first segment of the chunk: largest b with hkv * prefix[b] <= P0, then the kv head
  SegCursor first;
  {
    int lo_b = 0, hi_b = B;  // prefix[lo_b]*hkv <= P0 < prefix[hi_b]*hkv
    while (hi_b - lo_b > 1) {
      const int mid = (lo_b + hi_b) >> 1;
      if (prefix[mid] * hkv <= P0) lo_b = mid; else hi_b = mid;
    }
    first.b = lo_b;
    first.np = prefix[lo_b + 1] - prefix[lo_b];
    first.kvh = (P0 - prefix[lo_b] * hkv) / first.np;
    first.start = prefix[lo_b] * hkv + first.kvh * first.np;
  }

  if (warp == NC) {
    // ================= retiring warp =================
    // lane -> rows (8h + lane % 8), columns [32 * (lane / 8), +32)
    const int rr = lane & 7, d0 = 32 * (lane >> 3);
    int n_total = 0;
    {
      PieceWalker w;
      w.init(first, P0, P1, chunk);
      for (int g = P0; g < P1;) {
        const Piece q = w.at(g, prefix, hkv);
        n_total += q.solo() ? 0 : 1;
        g = q.e;
      }
    }
    PieceWalker walk;
    walk.init(first, P0, P1, chunk);
    int n = 0;
    for (int g = P0; g < P1;) {
      const Piece q = walk.at(g, prefix, hkv);
      g = q.e;
      if (q.solo()) continue;
      if (n == n_total - 1) break;  // the chunk's last shared piece is retired by the compute warps
      const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + q.kvh) : p.v_scale;
      named_sync(kBarReady, NT);  // the compute warps' sums for this piece are complete
      float acc[NH][32], big[NH], lt[NH];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const int row = 8 * h + rr;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          float4* cell = reinterpret_cast<float4*>(sm_acc) + acc_f4(row, (d0 >> 2) + t);
          const float4 x = *cell;
          acc[h][4 * t] = x.x * vs; acc[h][4 * t + 1] = x.y * vs;
          acc[h][4 * t + 2] = x.z * vs; acc[h][4 * t + 3] = x.w * vs;
          *cell = make_float4(0.f, 0.f, 0.f, 0.f);  // leave the buffer zeroed for the next piece
        }
        big[h] = -INFINITY;
        lt[h] = 0.f;
#pragma unroll
        for (int w = 0; w < NC; ++w) {
          big[h] = fmaxf(big[h], sm_m[w * ROWS + row]);
          lt[h] += sm_l[w * ROWS + row];
        }
        big[h] *= kLn2;
      }
      __threadfence_block();
      if (n + 1 < n_total) named_arrive(kBarFree, NT);  // buffer and sm_m/sm_l may be reused
      ++n;
      mark_phase(tp, 5, lane == 0);

      const int c_first = q.seg_start / chunk, c_last = (q.seg_start + q.np - 1) / chunk;
      const int pieces = c_last - c_first + 1;
      const int piece = (int)blockIdx.x - c_first;
      if (pieces > bp.workspace_splits) {  // cannot happen with the host's min_chunk; never write past the workspace
        if (lane == 0) atomicExch(tp.status, kErrWorkspace);
        continue;
      }
      bool last = false;
      if (pieces > 1) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const int row = 8 * h + rr;
          if (row < p.group) {
            const int hq = q.kvh * p.group + row;
            const int64_t pidx = (int64_t)q.b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h +
                                 (int64_t)piece * p.partial_stride_s;
            float* dst = reinterpret_cast<float*>(p.partial_output) + pidx * D + d0;
#pragma unroll
            for (int t = 0; t < 32; t += 4)
              *reinterpret_cast<float4*>(dst + t) = make_float4(acc[h][t], acc[h][t + 1], acc[h][t + 2], acc[h][t + 3]);
            if (d0 == 0) {
              p.partial_max[pidx] = big[h];
              p.partial_sum[pidx] = lt[h];
            }
          }
        }
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(bp.semaphores + q.b * hkv + q.kvh, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        last = old == pieces - 1;
        if (last) __threadfence();
      }
      if (pieces == 1 || last) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const int row = 8 * h + rr;
          if (row >= p.group) continue;
          const int hq = q.kvh * p.group + row;
          float m_nat = big[h], den = lt[h];
          if (last) {
            // Merge the other pieces into this CTA's own (still in registers), two pieces per
            // round trip: their maxima, sums and data are requested together.
            const int64_t pbase = (int64_t)q.b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h;
            const float* pout = reinterpret_cast<const float*>(p.partial_output);
            for (int s0 = 0; s0 < pieces - 1; s0 += 2) {
              float4 x[2][8];
              float ms[2], ls[2];
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                // the v-th other piece of this batch: indices skip this CTA's own piece
                int s = s0 + v;
                const bool on = s < pieces - 1;
                s = on ? (s >= piece ? s + 1 : s) : piece;
                const int64_t pidx = pbase + (int64_t)s * p.partial_stride_s;
                ms[v] = __ldcg(p.partial_max + pidx);
                ls[v] = __ldcg(p.partial_sum + pidx);
                if (!on) { ms[v] = -INFINITY; ls[v] = 0.f; }
                const float4* src = reinterpret_cast<const float4*>(pout + pidx * D + d0);
#pragma unroll
                for (int t = 0; t < 8; ++t) x[v][t] = __ldcg(src + t);
              }
              const float m_new = fmaxf(m_nat, fmaxf(ms[0], ms[1]));
              const float own = expf(m_nat - m_new);
              const float cf0 = expf(ms[0] - m_new), cf1 = expf(ms[1] - m_new);
              den = den * own + ls[0] * cf0 + ls[1] * cf1;
              m_nat = m_new;
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                acc[h][4 * t] = acc[h][4 * t] * own + cf0 * x[0][t].x + cf1 * x[1][t].x;
                acc[h][4 * t + 1] = acc[h][4 * t + 1] * own + cf0 * x[0][t].y + cf1 * x[1][t].y;
                acc[h][4 * t + 2] = acc[h][4 * t + 2] * own + cf0 * x[0][t].z + cf1 * x[1][t].z;
                acc[h][4 * t + 3] = acc[h][4 * t + 3] * own + cf0 * x[0][t].w + cf1 * x[1][t].w;
              }
            }
          }
          float lo16[16], hi16[16];
#pragma unroll
          for (int t = 0; t < 16; ++t) { lo16[t] = acc[h][t]; hi16[t] = acc[h][16 + t]; }
          store_row16<QBF16>(p, q.b, hq, d0, lo16, m_nat, den, d0 == 0);
          store_row16<QBF16>(p, q.b, hq, d0 + 16, hi16, m_nat, den, false);
        }
        if (last && lane == 0) bp.semaphores[q.b * hkv + q.kvh] = 0;  // ready for the next call
      }
      mark_phase(tp, 6, lane == 0);  // piece retired
    }
    return;
  }

  // ================= compute warps =================
  // ---- producer side: this warp's pairs in chunk order, each into the next ring stage
  struct PairRef { int32_t phys0, phys1, kvh; bool two, valid; };
  PieceWalker pwalk;
  pwalk.init(first, P0, P1, chunk);
  Piece pp = pwalk.at(P0, prefix, hkv);
  int px = piece_first(pp, warp);
  bool pdone = false;
  auto producer_settle = [&]() {  // move to the next piece in which this warp has a pair
    while (!pdone && px >= pp.e) {
      if (pp.e >= P1) { pdone = true; break; }
      pp = pwalk.at(pp.e, prefix, hkv);
      px = piece_first(pp, warp);
    }
  };
  producer_settle();
  auto locate = [&]() {  // page ids of this warp's next pair (global loads, all lanes alike)
    PairRef r;
    r.valid = !pdone;
    r.phys0 = r.phys1 = r.kvh = 0;
    r.two = false;
    if (!pdone) {
      const int page0 = page_first + 2 * (px - pp.seg_start);
      const int last_page = (lens[pp.b] - 1) / kPage;
      r.two = page0 + 1 <= last_page;
      r.kvh = pp.kvh;
      const int32_t* row = p.block_table + (int64_t)pp.b * p.bt_stride_b;
      r.phys0 = __ldg(row + page0);
      r.phys1 = r.two ? __ldg(row + page0 + 1) : 0;
      px += piece_stride(pp);
      producer_settle();
    }
    return r;
  };
  auto fire = [&](int k, const PairRef& r) {  // lane 0 only
    const uint32_t bar = my_bars + 8 * (k % NSTAGE);
    const uint32_t dst = my_ring + (k % NSTAGE) * kStage;
    mbar_expect_tx(bar, r.two ? kStage : kStage / 2);
    const int c1 = tp.head_is_dim1 ? r.kvh : 0;
    const int c2 = tp.head_is_dim1 ? 0 : r.kvh;
    tma_load_tile(dst, &tmap_k, bar, c1, c2, r.phys0);
    tma_load_tile(dst + 2 * kTile, &tmap_v, bar, c1, c2, r.phys0);
    if (r.two) {
      tma_load_tile(dst + kTile, &tmap_k, bar, c1, c2, r.phys1);
      tma_load_tile(dst + 3 * kTile, &tmap_v, bar, c1, c2, r.phys1);
    }
  };
  __syncwarp();
  PairRef pending;
  {
    PairRef r[NSTAGE + 1];
#pragma unroll
    for (int k = 0; k <= NSTAGE; ++k) r[k] = locate();
#pragma unroll
    for (int k = 0; k < NSTAGE; ++k)
      if (r[k].valid && lane == 0) fire(k, r[k]);
    pending = r[NSTAGE];
  }
  mark_phase(tp, 2);  // first copies issued
  int n_total_shared = 0;  // shared pieces of this chunk (same walk as the retiring warp's)
  {
    PieceWalker w;
    w.init(first, P0, P1, chunk);
    for (int gg = P0; gg < P1;) {
      const Piece t = w.at(gg, prefix, hkv);
      n_total_shared += t.solo() ? 0 : 1;
      gg = t.e;
    }
  }

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

  // ---- consumer side: the pieces this warp takes part in (shared ones, and its own solo ones),
  // in chunk order; the query of the next such piece is fetched while the current one retires
  PieceWalker cwalk;
  cwalk.init(first, P0, P1, chunk);
  int g = P0;
  auto next_piece = [&](Piece& q) {  // false when the chunk is exhausted
    while (g < P1) {
      q = cwalk.at(g, prefix, hkv);
      g = q.e;
      if (!q.solo() || q.owner == warp) return true;
    }
    return false;
  };
  BalState<NH> st;
  int cons = 0;      // pairs this warp has consumed
  int n_shared = 0;  // pieces reduced through shared memory so far
  bool ok = true;
  Piece q;
  bool have = next_piece(q);
  uint32_t qb[NH][8][2];
  if (have && piece_first(q, warp) < q.e) bal_load_q<QBF16, NH>(qb, p, q.b, q.kvh, i, j);
  bool first_piece = true;
  while (have) {
    const int x0 = piece_first(q, warp), stride = piece_stride(q);
    const int seq_len = lens[q.b];
    const float ks = p.k_scale_ph ? __ldg(p.k_scale_ph + q.kvh) : p.k_scale;
    const float scale_log2 = ks * p.sm_scale * kLog2e;
    bal_reset<NH>(st);
    for (int x = x0; ok && x < q.e; x += stride) {
      const int s = cons % NSTAGE;
      if (!mbar_wait_bounded(my_bars + 8 * s, (cons / NSTAGE) & 1)) { ok = false; break; }
      if (cons == 0) mark_phase(tp, 3);  // first data landed
      const int tok0 = (page_first + 2 * (x - q.seg_start)) * kPage;
      bal_step<NH>(st, my_ring + s * kStage, k_off, v_off, qb, scale_log2, tok0, p.kv_start, seq_len, i, j);
      // all reads of the stage fed MMAs above: hand it back to TMA for this warp's pair cons + NSTAGE
      __syncwarp();
      if (pending.valid) {
        if (lane == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          fire(cons + NSTAGE, pending);
        }
        pending = locate();
      }
      ++cons;
    }
    if (first_piece) mark_phase(tp, 4);  // (warp 0) streaming of its first piece done
    first_piece = false;

    // next piece and its query: the loads fly while this piece is reduced
    Piece nq;
    const bool have_next = next_piece(nq);
    uint32_t qn[NH][8][2];
    if (have_next && piece_first(nq, warp) < nq.e) bal_load_q<QBF16, NH>(qn, p, nq.b, nq.kvh, i, j);

    // ---- this warp's sums over the tokens it saw
    float lsum[NH][2];
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = st.l[h][e];
        x += __shfl_xor_sync(0xffffffffu, x, 4);
        x += __shfl_xor_sync(0xffffffffu, x, 8);
        x += __shfl_xor_sync(0xffffffffu, x, 16);
        lsum[h][e] = x;
      }
    if (q.solo()) {
      // a small whole segment: write its rows straight from registers
      const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + q.kvh) : p.v_scale;
#pragma unroll
      for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int row = 8 * h + 2 * j + e;
          if (row >= p.group) continue;
          float v[16];
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            v[2 * mt] = st.o[h][mt][e] * vs;
            v[2 * mt + 1] = st.o[h][mt][2 + e] * vs;
          }
          store_row16<QBF16>(p, q.b, q.kvh * p.group + row, 16 * i, v, st.m[h][e] * kLn2, lsum[h][e], i == 0);
        }
    } else {
      // ---- reduction over the compute warps in shared memory; the retiring warp takes it from there
      if (n_shared > 0) named_sync(kBarFree, NT);  // previous piece has been read out
#pragma unroll
      for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (i == 0) sm_m[warp * ROWS + 8 * h + 2 * j + e] = st.m[h][e];
      named_sync(kBarMax, NC * 32);
      float fac[NH][2];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        float f[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int row = 8 * h + 2 * j + e;
          float big = -INFINITY;
#pragma unroll
          for (int w = 0; w < NC; ++w) big = fmaxf(big, sm_m[w * ROWS + row]);
          f[e] = (st.m[h][e] == -INFINITY) ? 0.f : exp2f(st.m[h][e] - big);
          if (i == 0) sm_l[warp * ROWS + row] = lsum[h][e] * f[e];
        }
        fac[h][0] = f[0];
        fac[h][1] = f[1];
      }
      // Sum the four warps' O^T without atomics: in phase k warp w adds the quarter
      // (w + k) % 4 of its values (m-tiles 2q, 2q+1, i.e. columns 16i + 4q .. +3 of rows 2j, 2j+1)
      // with plain float4 read-modify-writes; no two warps touch the same quarter in a phase.
#pragma unroll
      for (int k = 0; k < NC; ++k) {
        const int qq = (warp + k) & (NC - 1);
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int row = 8 * h + 2 * j + e;
            float4* cell = reinterpret_cast<float4*>(sm_acc) + acc_f4(row, 4 * i + qq);
            float4 x = *cell;
            // m-tile 2q: columns +0 (c = e) and +1 (c = 2 + e); m-tile 2q+1: +2 and +3
            float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
#pragma unroll
            for (int z = 0; z < NC; ++z)
              if (z == qq) {
                v0 = st.o[h][2 * z][e]; v1 = st.o[h][2 * z][2 + e];
                v2 = st.o[h][2 * z + 1][e]; v3 = st.o[h][2 * z + 1][2 + e];
              }
            x.x += v0 * fac[h][e]; x.y += v1 * fac[h][e]; x.z += v2 * fac[h][e]; x.w += v3 * fac[h][e];
            *cell = x;
          }
        if (k + 1 < NC) named_sync(kBarMax, NC * 32);
      }
      __threadfence_block();
      if (n_shared + 1 < n_total_shared) {
        named_arrive(kBarReady, NT);
      } else {
        // The chunk's last shared piece decides when the CTA is done: all four compute warps
        // retire it together (8 columns per thread, every merge operand requested at once)
        // instead of queueing it behind the retiring warp's earlier pieces.
        named_sync(kBarMax, NC * 32);
        const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + q.kvh) : p.v_scale;
        const int c_first = q.seg_start / chunk, c_last = (q.seg_start + q.np - 1) / chunk;
        const int pieces = c_last - c_first + 1, piece = (int)blockIdx.x - c_first;
        const bool fits = pieces <= bp.workspace_splits;
        if (!fits && threadIdx.x == 0) atomicExch(tp.status, kErrWorkspace);
        constexpr int ITEMS = ROWS * 16 / (NC * 32);  // (row, 8 columns) slices per thread
        float a8[ITEMS][8], m_nat[ITEMS], den[ITEMS];
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int e = threadIdx.x + it * NC * 32, row = e >> 4, c8 = (e & 15) * 8;
          const float4 x0 = reinterpret_cast<const float4*>(sm_acc)[acc_f4(row, c8 >> 2)];
          const float4 x1 = reinterpret_cast<const float4*>(sm_acc)[acc_f4(row, (c8 >> 2) + 1)];
          a8[it][0] = x0.x * vs; a8[it][1] = x0.y * vs; a8[it][2] = x0.z * vs; a8[it][3] = x0.w * vs;
          a8[it][4] = x1.x * vs; a8[it][5] = x1.y * vs; a8[it][6] = x1.z * vs; a8[it][7] = x1.w * vs;
          float big = -INFINITY, lt = 0.f;
#pragma unroll
          for (int w = 0; w < NC; ++w) {
            big = fmaxf(big, sm_m[w * ROWS + row]);
            lt += sm_l[w * ROWS + row];
          }
          m_nat[it] = big * kLn2;
          den[it] = lt;
          if (fits && pieces > 1 && row < p.group) {
            const int hq = q.kvh * p.group + row;
            const int64_t pidx = (int64_t)q.b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h +
                                 (int64_t)piece * p.partial_stride_s;
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.partial_output) + pidx * D + c8);
            dst[0] = make_float4(a8[it][0], a8[it][1], a8[it][2], a8[it][3]);
            dst[1] = make_float4(a8[it][4], a8[it][5], a8[it][6], a8[it][7]);
            if (c8 == 0) {
              p.partial_max[pidx] = m_nat[it];
              p.partial_sum[pidx] = den[it];
            }
          }
        }
        bool last = false;
        if (fits && pieces > 1) {
          __threadfence();
          named_sync(kBarMax, NC * 32);
          if (threadIdx.x == 0) sm_misc[0] = atomicAdd(bp.semaphores + q.b * hkv + q.kvh, 1) == pieces - 1;
          named_sync(kBarMax, NC * 32);
          last = sm_misc[0] != 0;
          if (last) __threadfence();
        }
        if (fits && (pieces == 1 || last)) {
#pragma unroll
          for (int it = 0; it < ITEMS; ++it) {
            const int e = threadIdx.x + it * NC * 32, row = e >> 4, c8 = (e & 15) * 8;
            if (row >= p.group) continue;
            const int hq = q.kvh * p.group + row;
            if (last) {
              const int64_t pbase = (int64_t)q.b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h;
              const float* pout = reinterpret_cast<const float*>(p.partial_output);
              for (int s0 = 0; s0 < pieces - 1; s0 += 8) {
                float4 x[8][2];
                float ms[8], ls[8];
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  int sidx = s0 + v;
                  const bool on = sidx < pieces - 1;
                  sidx = on ? (sidx >= piece ? sidx + 1 : sidx) : piece;
                  const int64_t pidx = pbase + (int64_t)sidx * p.partial_stride_s;
                  ms[v] = __ldcg(p.partial_max + pidx);
                  ls[v] = __ldcg(p.partial_sum + pidx);
                  if (!on) { ms[v] = -INFINITY; ls[v] = 0.f; }
                  const float4* src = reinterpret_cast<const float4*>(pout + pidx * D + c8);
                  x[v][0] = __ldcg(src);
                  x[v][1] = __ldcg(src + 1);
                }
                float m_new = m_nat[it];
#pragma unroll
                for (int v = 0; v < 8; ++v) m_new = fmaxf(m_new, ms[v]);
                const float own = expf(m_nat[it] - m_new);
                den[it] *= own;
#pragma unroll
                for (int t = 0; t < 8; ++t) a8[it][t] *= own;
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  const float cf = expf(ms[v] - m_new);
                  den[it] += ls[v] * cf;
                  a8[it][0] += cf * x[v][0].x; a8[it][1] += cf * x[v][0].y;
                  a8[it][2] += cf * x[v][0].z; a8[it][3] += cf * x[v][0].w;
                  a8[it][4] += cf * x[v][1].x; a8[it][5] += cf * x[v][1].y;
                  a8[it][6] += cf * x[v][1].z; a8[it][7] += cf * x[v][1].w;
                }
                m_nat[it] = m_new;
              }
            }
            if (p.packed_output != nullptr) {
              float* dst = p.packed_output + ((int64_t)q.b * p.num_q_heads + hq) * (D + 2);
#pragma unroll
              for (int t = 0; t < 8; t += 2) *reinterpret_cast<float2*>(dst + c8 + t) = make_float2(a8[it][t], a8[it][t + 1]);
              if (c8 == 0) { dst[D] = m_nat[it]; dst[D + 1] = den[it]; }
            } else {
              const float inv = 1.f / den[it];
              uint32_t wv[4];
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                if constexpr (QBF16) {
                  __nv_bfloat162 x = __floats2bfloat162_rn(a8[it][2 * t] * inv, a8[it][2 * t + 1] * inv);
                  wv[t] = *reinterpret_cast<uint32_t*>(&x);
                } else {
                  wv[t] = pack_f16x2(a8[it][2 * t] * inv, a8[it][2 * t + 1] * inv);
                }
              }
              uint16_t* dst = reinterpret_cast<uint16_t*>(p.output) + (int64_t)q.b * p.o_stride_b + (int64_t)hq * p.o_stride_h + c8;
              *reinterpret_cast<uint2*>(dst) = make_uint2(wv[0], wv[1]);
              *reinterpret_cast<uint2*>(dst + 4) = make_uint2(wv[2], wv[3]);
            }
          }
          if (last && threadIdx.x == 0) bp.semaphores[q.b * hkv + q.kvh] = 0;  // ready for the next call
        }
        mark_phase(tp, 6);  // chunk's last shared piece retired
      }
      ++n_shared;
    }
    q = nq;
    have = have_next;
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
      for (int t = 0; t < 8; ++t) { qb[h][t][0] = qn[h][t][0]; qb[h][t][1] = qn[h][t][1]; }
  }
  if (!ok && lane == 0) {
    // a copy never landed: record it; give the copies still in flight a bounded chance to land
    atomicExch(tp.status, kErrTmaTimeout);
    for (int u = cons + 1; u < cons + NSTAGE; ++u) mbar_wait_bounded(my_bars + 8 * (u % NSTAGE), (u / NSTAGE) & 1);
  }
}

}  // namespace pfd
