// Device code of the paged FP8-e4m3 KV GQA decode-attention path for sm_100a.
//
// Work item = (KV split, kv head, sequence).  All g = Hq/Hkv query heads of the group are
// rows of one 16-row MMA tile, so every K/V byte is fetched once per group (the reference
// kernels launch one program per *query* head and re-read the cache g times:
// integrations/vllm/cuda/l20_paged_decode.cu:308-311, l20_paged_split_kv.py:164-168).
//
// Per warp and per 16-token page:
//   S = Q K^T   : mma.sync.m16n8k16 f16 -> f32.  e4m3 -> f16 is exact (cvt.rn.f16x2.e4m3x2);
//                 a dot product does not care about the order of d, so Q's A-fragments are
//                 permuted once such that every thread's natural 16-byte K load *is* its
//                 B-fragment.  k_scale * sm_scale * log2(e) is applied to the 8 scores, not
//                 to the bytes.
//   online softmax in fp32 (exp2), row max over the quad with two shuffles.
//   O += P V    : same MMA; the token-pair interleave V needs is two byte permutes per word.
// Warps of a CTA take pages round-robin and never synchronise inside the loop; they merge
// their (m, l, O) once at the end through shared memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pfd {

constexpr int kPage = 16;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct KernelParams {
  const void* __restrict__ query;
  const uint8_t* __restrict__ key_cache;
  const uint8_t* __restrict__ value_cache;
  const int32_t* __restrict__ block_table;
  const int32_t* __restrict__ seq_lens;
  const int32_t* __restrict__ page_indptr;  // optional: block_table is then a flat list, row b starts at page_indptr[b]
  const float* __restrict__ k_scale_ph;
  const float* __restrict__ v_scale_ph;
  void* partial_output;
  float* partial_max;
  float* partial_sum;
  void* output;
  float* packed_output;
  int64_t q_stride_b, q_stride_h;
  int64_t k_stride_page, k_stride_token, k_stride_head;
  int64_t v_stride_page, v_stride_token, v_stride_head;
  int64_t bt_stride_b;
  int64_t partial_stride_b, partial_stride_h, partial_stride_s;
  int64_t o_stride_b, o_stride_h;
  float k_scale, v_scale, sm_scale;
  int32_t num_q_heads, num_kv_heads, group;
  int32_t split_size, kv_start;
  int32_t partial_dtype;
  int32_t direct_out;  // 1: a sequence with a single split writes its final result itself
  int32_t bt_cols;     // width of a block-table row
  int32_t slot_offset; // workspace slots [0, slot_offset) are filled by another kernel (dense prefix pass)
  // Grouped shared-prefix decode: row b attends from token row_kv_start[b] & ~15 on (the prefix of
  // its group, 0 for a request in no group) and owns ceil(that / 256) of the slots in front.
  const int32_t* row_kv_start;
  int32_t row_kv_cap;  // upper bound applied to row_kv_start (a multiple of 16): the slots in front cover no more
  int32_t split_size_loner;  // grouped decode: split size of a request in no group (it attends from 0); 0 = split_size
  int32_t early_metadata;  // 1: seq_lens and block_table may be read before the preceding kernel has completed
  int32_t early_kv;        // 1: so may K/V pages, except each sequence's last (balanced kernel with a plan)
  int32_t kv_evict_first;  // 1: K/V tiles are loaded with the L2 evict-first hint
  // KV-range exchange (xch_world > 0): the packed (o, m, l) rows of this rank go, instead of to
  // packed_output, into slot xch_rank of every rank's receive buffer [2][world][rows][kXchRow]
  // (8-byte words) with plain stores over NVLink.  Every word carries its value in the low and
  // the step's tag in the high half, and an aligned 8-byte store arrives whole: the receiver
  // polls the words themselves, so no fence, flag or counter is needed (the low-latency
  // protocol of collective libraries).  The step's tag is device-resident (a replayed CUDA
  // graph carries no per-step arguments): xch_control[0] counts the completed steps, the tag is
  // that count + 1 and its lowest bit picks the half of the buffers.
  int32_t xch_world, xch_rank, xch_rows;
  unsigned long long* xch_recv[8];
  uint32_t* xch_control;   // local: [0] steps completed, [1] merge CTAs done
#ifdef PFD_BOUNDS_CHECK
  int64_t dbg_ws_rows;     // self-checking builds: rows of the workspace, sequences of the batch
  int32_t dbg_batch;
#endif
};

// Programmatic dependent launch: the split-KV partial kernel lets its dependent (the merge
// kernel, launched with the programmatic-serialization attribute) be scheduled while it is
// still running; the merge kernel reads seq_lens, then waits here until the whole partial grid
// has completed and its memory is visible.  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- KV-range exchange: where packed rows go, and the hand-over to the other ranks ----------
// A row of a receive buffer: o[128], m, l, one tagged 8-byte word each.
constexpr int kXchRow = 130;
__device__ __forceinline__ unsigned long long xch_word(float v, uint32_t tag) {
  return (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
}
__device__ __forceinline__ void xch_store2(unsigned long long* p, float a, float b, uint32_t tag) {
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(xch_word(a, tag)), "l"(xch_word(b, tag))
               : "memory");
}
// Two tagged words; false while either has not arrived.
__device__ __forceinline__ bool xch_load2(const unsigned long long* p, uint32_t tag, float& a, float& b) {
  unsigned long long x, y;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(x), "=l"(y) : "l"(p) : "memory");
  a = __uint_as_float((uint32_t)x);
  b = __uint_as_float((uint32_t)y);
  return (uint32_t)(x >> 32) == tag && (uint32_t)(y >> 32) == tag;
}
// Tag of the exchange step this grid belongs to (0 without an exchange).  Read it after the
// grid's programmatic-dependency wait: the previous step's merge kernel advances the count.
__device__ __forceinline__ uint32_t exchange_step(const KernelParams& p) {
  return p.xch_world > 0 ? __ldcg(p.xch_control) + 1u : 0u;
}
__device__ __forceinline__ unsigned long long* xch_row(const KernelParams& p, int dest, int64_t row, uint32_t step) {
  return p.xch_recv[dest] + (((int64_t)(step & 1u) * p.xch_world + p.xch_rank) * p.xch_rows + row) * kXchRow;
}

// The one address function every kernel uses for "which cache slot holds token t of
// sequence b".  Returns the physical page; the slot is page * 16 + t % 16.
// First token the split-KV kernels attend for sequence b.
__device__ __forceinline__ int kv_start_of(const KernelParams& p, int b) {
  return p.row_kv_start != nullptr ? min(__ldg(p.row_kv_start + b) & ~15, p.row_kv_cap) : p.kv_start;
}

// Split size of sequence b, whose first attended token is kv0: in a grouped decode a request in
// no group has the whole context to cover with the same number of splits as the others' suffixes.
__device__ __forceinline__ int split_size_of(const KernelParams& p, int kv0) {
  return (p.row_kv_start != nullptr && kv0 == 0 && p.split_size_loner > 0) ? p.split_size_loner : p.split_size;
}

__device__ __forceinline__ int32_t page_of(const int32_t* __restrict__ block_table,
                                           int64_t bt_stride_b, int b, int logical_page) {
  return __ldg(block_table + (int64_t)b * bt_stride_b + logical_page);
}

__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((uint16_t)two_bytes));
  return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc_16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_8(const uint8_t* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Which token row of a page sits in column n of an 8-column score tile.  Any bijection works
// for the maths (P's columns and V's rows follow it); this one makes both the K and the V
// shared-memory reads of the TMA kernel bank-conflict free under the 128-byte swizzle:
// columns 2q and 2q+1 land on rows that differ in bit 2, and the rows of the even (odd)
// columns differ pairwise in bits 1..2.  rho = [0, 5, 2, 7, 4, 1, 6, 3].
__device__ __forceinline__ int rho(int n) { return (n & 6) ^ ((n & 1) * 5); }

// Register image of one (page, kv head) tile as the MMA fragments want it.
//   K: thread (i = lane/4, j = lane%4) holds bytes [16*(j+4l), +16) of rows rho(i), 8 + rho(i).
//   V: the same thread holds bytes [CB*i, +CB) (CB = D/8) of rows 2j, 2j^5, 8+2j, 8+(2j^5),
//      i.e. the rows of its own score columns 2j and 2j+1 in both column tiles.
__device__ __forceinline__ int v_row(int j, int r) { return ((r & 1) ? ((2 * j) ^ 5) : 2 * j) + 8 * (r >> 1); }
template <int D>
struct TileRegs {
  static constexpr int KL = D / 64;  // 16-byte K chunks per thread per row
  static constexpr int VW = D / 32;  // 32-bit V words per thread per row
  uint32_t k[2][KL][4];
  uint32_t v[4][VW];
};

template <int D>
__device__ __forceinline__ void load_tile_global(TileRegs<D>& t, const uint8_t* kpage,
                                                 const uint8_t* vpage, int64_t kst, int64_t vst,
                                                 int i, int j) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int l = 0; l < TileRegs<D>::KL; ++l) {
      uint4 x = ldg_nc_16(kpage + (int64_t)(nt * 8 + rho(i)) * kst + 16 * (j + 4 * l));
      t.k[nt][l][0] = x.x; t.k[nt][l][1] = x.y; t.k[nt][l][2] = x.z; t.k[nt][l][3] = x.w;
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint8_t* p = vpage + (int64_t)v_row(j, r) * vst + (D / 8) * i;
    if constexpr (D == 128) {
      uint4 x = ldg_nc_16(p);
      t.v[r][0] = x.x; t.v[r][1] = x.y; t.v[r][2] = x.z; t.v[r][3] = x.w;
    } else {
      uint2 x = ldg_nc_8(p);
      t.v[r][0] = x.x; t.v[r][1] = x.y;
    }
  }
}

// Per-warp running state: rows i (index 0) and i+8 (index 1) of the 16-row head tile.
template <int D>
struct WarpState {
  float o[D / 8][4];  // n-tile m covers d = 32j + 16e + m (D=128) / 16j + 8e + m (D=64)
  float m[2];         // running max, log2 domain
  float l[2];         // running sum, this thread's columns only (quad-reduced at the end)
};

// ---- the three phases of one 16-token tile ------------------------------------------------
// tok0 = global token index of row 0 of the page; tokens outside [lo, hi) are masked.

// S = Q K^T for NT 8-column tiles (raw, unscaled); k-steps outermost so that consecutive MMAs
// belong to independent accumulators.
template <int D, int NT>
__device__ __forceinline__ void qk_scores(float (&s)[NT][4], const uint32_t (&k)[NT][D / 64][4],
                                          const uint32_t (&qa)[D / 16][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int l = 0; l < D / 64; ++l) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint32_t word = k[nt][l][w];
        mma_m16n8k16(s[nt], qa[l * 4 + w], cvt_e4m3x2_to_f16x2(word),
                     cvt_e4m3x2_to_f16x2(word >> 16));
      }
    }
  }
}

// Scale, mask, online softmax over NT/2 pages; rescales O and returns P as the f16 A-fragments
// of the PV MMAs (pa[t] for page t).  Column tile nt covers tokens tok0 + 8*nt + rho(.).
template <int D, int NT>
__device__ __forceinline__ void softmax_step(WarpState<D>& st, float (&s)[NT][4],
                                             uint32_t (&pa)[NT / 2][4], float scale_log2, bool edge,
                                             int tok0, int lo, int hi, int j) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float x = s[nt][c] * scale_log2;
      if (edge) {
        const int tok = tok0 + nt * 8 + rho(2 * j + (c & 1));
        if (tok < lo || tok >= hi) x = -INFINITY;
      }
      s[nt][c] = x;
    }
  }
  float mx0 = fmaxf(s[0][0], s[0][1]), mx1 = fmaxf(s[0][2], s[0][3]);
#pragma unroll
  for (int nt = 1; nt < NT; ++nt) {
    mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
    mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m[0], mx0);
  const float mn1 = fmaxf(st.m[1], mx1);
  const float alpha0 = exp2f(st.m[0] - mn0);
  const float alpha1 = exp2f(st.m[1] - mn1);
  st.m[0] = mn0;
  st.m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const float p0 = exp2f(s[nt][0] - mn0), p1 = exp2f(s[nt][1] - mn0);
    const float p2 = exp2f(s[nt][2] - mn1), p3 = exp2f(s[nt][3] - mn1);
    sum0 += p0 + p1;
    sum1 += p2 + p3;
    pa[nt >> 1][(nt & 1) * 2 + 0] = pack_f16x2(p0, p1);
    pa[nt >> 1][(nt & 1) * 2 + 1] = pack_f16x2(p2, p3);
  }
  st.l[0] = st.l[0] * alpha0 + sum0;
  st.l[1] = st.l[1] * alpha1 + sum1;
  // the running max rarely moves after the first tiles: skip the 4*D/8 multiplies then
  if (__any_sync(0xffffffffu, (alpha0 != 1.f) | (alpha1 != 1.f))) {
#pragma unroll
    for (int m = 0; m < D / 8; ++m) {
      st.o[m][0] *= alpha0; st.o[m][1] *= alpha0;
      st.o[m][2] *= alpha1; st.o[m][3] *= alpha1;
    }
  }
}

// O += P V.  On edge pages the rows of tokens outside the range are zeroed first: their bytes
// may be anything (NaN patterns included) and 0 * NaN would poison the accumulator -- the
// reference's masked loads (`other=0.0`) do the same.
template <int D>
__device__ __forceinline__ void pv_accumulate(WarpState<D>& st, uint32_t (&v)[4][D / 32],
                                              const uint32_t (&pa)[4], bool edge, int tok0, int lo,
                                              int hi, int j) {
  if (edge) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int tok = tok0 + v_row(j, r);
      if (tok < lo || tok >= hi) {
#pragma unroll
        for (int w = 0; w < D / 32; ++w) v[r][w] = 0u;
      }
    }
  }
#pragma unroll
  for (int w = 0; w < D / 32; ++w) {
    // the two rows of each k-pair: interleave them byte-wise
    const uint32_t x01 = prmt(v[0][w], v[1][w], 0x5140u);
    const uint32_t y01 = prmt(v[0][w], v[1][w], 0x7362u);
    const uint32_t x23 = prmt(v[2][w], v[3][w], 0x5140u);
    const uint32_t y23 = prmt(v[2][w], v[3][w], 0x7362u);
    mma_m16n8k16(st.o[4 * w + 0], pa, cvt_e4m3x2_to_f16x2(x01), cvt_e4m3x2_to_f16x2(x23));
    mma_m16n8k16(st.o[4 * w + 1], pa, cvt_e4m3x2_to_f16x2(x01 >> 16), cvt_e4m3x2_to_f16x2(x23 >> 16));
    mma_m16n8k16(st.o[4 * w + 2], pa, cvt_e4m3x2_to_f16x2(y01), cvt_e4m3x2_to_f16x2(y23));
    mma_m16n8k16(st.o[4 * w + 3], pa, cvt_e4m3x2_to_f16x2(y01 >> 16), cvt_e4m3x2_to_f16x2(y23 >> 16));
  }
}

template <int D>
__device__ __forceinline__ void consume_tile(WarpState<D>& st, TileRegs<D>& t,
                                             const uint32_t (&qa)[D / 16][4], float scale_log2,
                                             int tok0, int lo, int hi, int j) {
  float s[2][4];
  uint32_t pa[1][4];
  const bool edge = (tok0 < lo) | (tok0 + kPage > hi);
  qk_scores<D, 2>(s, t.k, qa);
  softmax_step<D, 2>(st, s, pa, scale_log2, edge, tok0, lo, hi, j);
  pv_accumulate<D>(st, t.v, pa[0], edge, tok0, lo, hi, j);
}

// Q rows i and i+8 of the kv head's group as f16 A-fragments, d permuted to match the K loads:
// k-step ks = 4l + w covers d = 16*(j+4l) + 4w + {0,1 | 2,3}.
template <int D, bool QBF16>
__device__ __forceinline__ void load_q_frags(uint32_t (&qa)[D / 16][4], const KernelParams& p, int b,
                                             int kvh, int i, int j) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = i + 8 * half;
    const bool live = row < p.group;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(p.query) + (int64_t)b * p.q_stride_b +
                        (int64_t)(kvh * p.group + (live ? row : 0)) * p.q_stride_h;
#pragma unroll
    for (int l = 0; l < D / 64; ++l) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint2 raw = make_uint2(0u, 0u);
        if (live) raw = *reinterpret_cast<const uint2*>(q + 16 * (j + 4 * l) + 4 * w);
        uint32_t lo = raw.x, hi = raw.y;
        if constexpr (QBF16) {
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          lo = pack_f16x2(__bfloat162float(a.x), __bfloat162float(a.y));
          hi = pack_f16x2(__bfloat162float(c.x), __bfloat162float(c.y));
        }
        qa[l * 4 + w][half] = lo;       // a0 / a1 : k = 2j, 2j+1
        qa[l * 4 + w][2 + half] = hi;   // a2 / a3 : k = 2j+8, 2j+9
      }
    }
  }
}

__device__ __forceinline__ void store_partial_elem4(void* base, int dtype, int64_t idx, float4 v) {
  if (dtype == 0) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx) = v;
  } else if (dtype == 1) {
    __half2 a = __floats2half2_rn(v.x, v.y), c = __floats2half2_rn(v.z, v.w);
    uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(base) + idx) = u;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), c = __floats2bfloat162_rn(v.z, v.w);
    uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&c));
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = u;
  }
}

__device__ __forceinline__ float load_partial_elem(const void* base, int dtype, int64_t idx) {
  if (dtype == 0) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == 1) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

template <bool BF16>
__device__ __forceinline__ void store_out_elem4(void* base, int64_t idx, float4 v) {
  store_partial_elem4(base, BF16 ? 2 : 1, idx, v);
}

// Cross-warp merge + store, shared by the global-load and the TMA kernels.
//   sm_m/sm_l : [NWARPS][16], sm_o : [NWARPS][16][D] floats.
template <int D, bool QBF16, int NWARPS>
__device__ __forceinline__ void cta_merge_and_store(WarpState<D>& st, const KernelParams& p, int b,
                                                    int kvh, int split, int nsplits_seq,
                                                    float v_scale, float* sm_m, float* sm_l,
                                                    float* sm_o) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, i = lane >> 2, j = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
  }
  if (j == 0) {
    sm_m[warp * 16 + i] = st.m[0];
    sm_m[warp * 16 + i + 8] = st.m[1];
  }
  __syncthreads();
  float big[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) {
    big[0] = fmaxf(big[0], sm_m[w * 16 + i]);
    big[1] = fmaxf(big[1], sm_m[w * 16 + i + 8]);
  }
  // a warp that saw no tile has m = -inf, l = 0, o = 0: factor 0
  const float f0 = (st.m[0] == -INFINITY) ? 0.f : exp2f(st.m[0] - big[0]);
  const float f1 = (st.m[1] == -INFINITY) ? 0.f : exp2f(st.m[1] - big[1]);
  if (j == 0) {
    sm_l[warp * 16 + i] = st.l[0] * f0;
    sm_l[warp * 16 + i + 8] = st.l[1] * f1;
  }
  // Thread (i, j) owns d = (D/4)*j + (D/8)*e + m of rows i and i+8: as float4 chunks
  // q = (D/16)*j + (D/32)*e + m/4.  The chunk index is XOR-swizzled with (j + 4*(i&1)) so that
  // the eight lanes of a store phase hit eight different 16-byte bank groups.
  constexpr int CB = D / 8;
  const int swz = (D == 128) ? ((j + 4 * (i & 1)) & 7) : 0;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
#pragma unroll
    for (int m4 = 0; m4 < CB / 4; ++m4) {
      const int q = ((D / 16) * j + (D / 32) * e + m4) ^ swz;
      *reinterpret_cast<float4*>(sm_o + (warp * 16 + i) * D + 4 * q) =
          make_float4(st.o[4 * m4][e] * f0, st.o[4 * m4 + 1][e] * f0, st.o[4 * m4 + 2][e] * f0,
                      st.o[4 * m4 + 3][e] * f0);
      *reinterpret_cast<float4*>(sm_o + (warp * 16 + i + 8) * D + 4 * q) =
          make_float4(st.o[4 * m4][2 + e] * f1, st.o[4 * m4 + 1][2 + e] * f1,
                      st.o[4 * m4 + 2][2 + e] * f1, st.o[4 * m4 + 3][2 + e] * f1);
    }
  }
  __syncthreads();
  const bool direct = p.direct_out && nsplits_seq == 1;
  // g rows x D columns, 4 columns per thread-iteration
  for (int e = threadIdx.x; e < p.group * (D / 4); e += NWARPS * 32) {
    const int row = e / (D / 4), c4 = (e % (D / 4)) * 4;
    const int ql = c4 >> 2;
    const int qs = (D == 128) ? (ql ^ (((ql >> 3) + 4 * (row & 1)) & 7)) : ql;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float lsum = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(sm_o + (w * 16 + row) * D + 4 * qs);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      lsum += sm_l[w * 16 + row];
    }
    float big_row = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) big_row = fmaxf(big_row, sm_m[w * 16 + row]);
    acc.x *= v_scale; acc.y *= v_scale; acc.z *= v_scale; acc.w *= v_scale;
    const int hq = kvh * p.group + row;
    if (direct) {
      if (p.packed_output != nullptr) {
        float* dst = p.packed_output + ((int64_t)b * p.num_q_heads + hq) * (D + 2);
        dst[c4] = acc.x; dst[c4 + 1] = acc.y; dst[c4 + 2] = acc.z; dst[c4 + 3] = acc.w;
        if (c4 == 0) { dst[D] = big_row * kLn2; dst[D + 1] = lsum; }
      } else {
        const float inv = 1.f / lsum;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        store_out_elem4<QBF16>(p.output, (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h + c4, acc);
      }
    } else {
      const int64_t pidx = (int64_t)b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h +
                           (int64_t)(split + p.slot_offset) * p.partial_stride_s;
      store_partial_elem4(p.partial_output, p.partial_dtype, pidx * D + c4, acc);
      if (c4 == 0) {
        p.partial_max[pidx] = big_row * kLn2;
        p.partial_sum[pidx] = lsum;
      }
    }
  }
}

// Rows of a (sequence, kv head) with nothing to attend (seq_len <= kv_start), written by the
// partial kernel when no merge kernel follows (one split, direct output): zeros, or (0, -inf, 0)
// in packed form -- what the merge kernel writes for such rows when it does run.
template <int D>
__device__ __forceinline__ void write_empty_rows(const KernelParams& p, int b, int kvh) {
  for (int e = threadIdx.x; e < p.group * D; e += blockDim.x) {
    const int hq = kvh * p.group + e / D, d = e % D;
    if (p.packed_output != nullptr) {
      float* dst = p.packed_output + ((int64_t)b * p.num_q_heads + hq) * (D + 2);
      dst[d] = 0.f;
      if (d == 0) { dst[D] = -INFINITY; dst[D + 1] = 0.f; }
    } else {
      reinterpret_cast<uint16_t*>(p.output)[(int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h + d] = 0;
    }
  }
}

// Split-KV partial kernel, plain global loads (any 16-byte-aligned strides).
// grid = (splits, kv heads, sequences), block = NWARPS * 32.
template <int D, bool QBF16, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
paged_decode_fp8_partial_ldg_kernel(const KernelParams p) {
  pdl_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int seq_len = p.seq_lens[b];
  const int kv0 = kv_start_of(p, b);
  const int split_sz = split_size_of(p, kv0);
  const int lo = kv0 + split * split_sz;
  const int hi = min(lo + split_sz, seq_len);
  if (lo >= hi) {  // the merge kernel derives the live split count from seq_len
    pdl_wait();
    if (split == 0 && gridDim.x == 1 && p.direct_out) write_empty_rows<D>(p, b, kvh);
    return;
  }
  const int nsplits_seq = (seq_len - kv0 + split_sz - 1) / split_sz;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, i = lane >> 2, j = lane & 3;

  __shared__ float sm_m[NWARPS * 16];
  __shared__ float sm_l[NWARPS * 16];
  __shared__ __align__(16) float sm_o[NWARPS * 16 * D];

  uint32_t qa[D / 16][4];
  load_q_frags<D, QBF16>(qa, p, b, kvh, i, j);
  const float ks = p.k_scale_ph ? __ldg(p.k_scale_ph + kvh) : p.k_scale;
  const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + kvh) : p.v_scale;
  const float scale_log2 = ks * p.sm_scale * kLog2e;

  WarpState<D> st;
#pragma unroll
  for (int m = 0; m < D / 8; ++m) st.o[m][0] = st.o[m][1] = st.o[m][2] = st.o[m][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

  const int page_first = lo / kPage, page_last = (hi - 1) / kPage;
  const uint8_t* kbase = p.key_cache + (int64_t)kvh * p.k_stride_head;
  const uint8_t* vbase = p.value_cache + (int64_t)kvh * p.v_stride_head;

  TileRegs<D> cur, nxt;
  int pg = page_first + warp;
  if (pg <= page_last) {
    const int64_t phys = page_of(p.block_table, p.bt_stride_b, b, pg);
    load_tile_global<D>(cur, kbase + phys * p.k_stride_page, vbase + phys * p.v_stride_page,
                        p.k_stride_token, p.v_stride_token, i, j);
  }
  for (; pg <= page_last; pg += NWARPS) {
    const int pn = pg + NWARPS;
    if (pn <= page_last) {
      const int64_t phys = page_of(p.block_table, p.bt_stride_b, b, pn);
      load_tile_global<D>(nxt, kbase + phys * p.k_stride_page, vbase + phys * p.v_stride_page,
                          p.k_stride_token, p.v_stride_token, i, j);
    }
    consume_tile<D>(st, cur, qa, scale_log2, pg * kPage, lo, hi, j);
    cur = nxt;
  }
  cta_merge_and_store<D, QBF16, NWARPS>(st, p, b, kvh, split, nsplits_seq, vs, sm_m, sm_l, sm_o);
  pdl_wait();  // see the TMA kernel
}

// ---- TMA pipeline ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up when `limit_ns` nanoseconds (by %globaltimer) have passed, or after
// kSpinLimit rounds of polls whatever the clock says, so that a copy that never lands cannot
// hang the GPU; the caller records an error and carries on.
constexpr uint32_t kSpinLimit = 1u << 24;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned long long limit_ns) {
  // the common case costs nothing but polls: the clock is first read after 64 of them
#pragma unroll 1
  for (int k = 0; k < 64; ++k)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t round = 0; round < kSpinLimit; ++round) {
#pragma unroll 1
    for (int k = 0; k < 32; ++k)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
  return false;
}
// 4-D tiled TMA load of one (page, kv head) tile: CTA-local destination, every CTA issues its own copies.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const void* tmap, uint32_t bar, int c1,
                                              int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// The same load with an L2 eviction-priority hint.  K/V bytes are read once per step: marked
// evict-first they do not push the step's small reused data (query rows, block table, the
// partial results the merge kernel reads back) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const void* tmap, uint32_t bar, int c1,
                                              int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}

// The same two loads with an explicit innermost coordinate (in elements of the tensor map).
__device__ __forceinline__ void tma_load_tile_x(uint32_t dst, const void* tmap, uint32_t bar, int x, int c1,
                                                int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_tile_x(uint32_t dst, const void* tmap, uint32_t bar, int x, int c1,
                                                int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint4 lds_16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// Self-test of the bounded wait: one warp arms a barrier for bytes that no copy will ever
// deliver and waits; the wait must give up after limit_ns and set the error word.
__global__ void bounded_wait_selftest_kernel(int32_t* status, unsigned long long limit_ns, unsigned long long* waited_ns);

struct TmaParams {
  int32_t head_is_dim1;  // 1: tensor-map dims are (D, head, token, page); 0: (D, token, head, page)
  int32_t* status;       // device error word (0 = ok)
  unsigned long long wait_limit_ns;  // after this long a wait for a copy gives up and sets the error word
  unsigned long long* phase_times;  // [slots][8] nanosecond stamps; read only in builds with PFD_PHASE_STAMPS
};

// Tuning aid, compiled in only with -DPFD_PHASE_STAMPS (the shipped library leaves it out): the
// leader lane stores a %globaltimer stamp of phase k into phase_times[slot][k].
__device__ __forceinline__ void mark_phase_at(const TmaParams& tp, int slot, int k, bool leader) {
#ifdef PFD_PHASE_STAMPS
  if (tp.phase_times != nullptr && leader) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    tp.phase_times[(size_t)slot * 8 + k] = t;
  }
#else
  (void)tp; (void)slot; (void)k; (void)leader;
#endif
}
__device__ __forceinline__ void mark_value_at(const TmaParams& tp, int slot, int k, bool leader, unsigned long long v) {
#ifdef PFD_PHASE_STAMPS
  if (tp.phase_times != nullptr && leader) tp.phase_times[(size_t)slot * 8 + k] = v;
#else
  (void)tp; (void)slot; (void)k; (void)leader; (void)v;
#endif
}
// Tuning builds only: marks of kernels that carry no TmaParams (slot rows of the same buffer).
#ifdef PFD_PHASE_STAMPS
__device__ unsigned long long* g_dbg_stamps = nullptr;
#endif
__device__ __forceinline__ void dbg_mark(int slot, int k, bool leader) {
#ifdef PFD_PHASE_STAMPS
  if (g_dbg_stamps != nullptr && leader) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_dbg_stamps[(size_t)slot * 8 + k] = t;
    if (k == 0) { unsigned r; asm volatile("mov.u32 %0, %%smid;" : "=r"(r)); g_dbg_stamps[(size_t)slot * 8 + 7] = r + 1; }
  }
#else
  (void)slot; (void)k; (void)leader;
#endif
}
__device__ __forceinline__ unsigned sm_id() {
  unsigned r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}

constexpr int kErrTmaTimeout = 1;
constexpr int kErrSuffixBound = 5;  // grouped decode: a request's suffix exceeds the caller's bound

__global__ void bounded_wait_selftest_kernel(int32_t* status, unsigned long long limit_ns, unsigned long long* waited_ns) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar, 16);  // the arrival is in, the 16 bytes never come
  }
  __syncwarp();
  const unsigned long long t0 = global_timer_ns();
  const bool ok = mbar_wait_bounded(bar, 0, limit_ns);
  if (threadIdx.x == 0) {
    if (!ok) atomicExch(status, kErrTmaTimeout);
    if (waited_ns != nullptr) *waited_ns = global_timer_ns() - t0;
  }
}

// Split-KV partial kernel for head_dim 128, K/V tiles staged by TMA.
//
// Every warp owns a private ring of NSTAGE stages and one mbarrier per stage.  A stage holds
// two consecutive pages (32 tokens): [K0][K1][V0][V1], each tile [16][128] bytes, 128-byte
// swizzled and 1 KiB aligned (8 KiB per stage).  Lane 0 issues the tiled TMA loads of the
// warp's next page pair as soon as the warp has consumed a stage; warps never synchronise with
// each other inside the loop, and the bytes in flight do not cost registers.  Two pages per
// step give four independent QK^T accumulator chains and halve the per-token cost of the
// softmax bookkeeping (shuffles, rescale).
template <bool QBF16, int NWARPS, int NSTAGE>
__global__ void __launch_bounds__(NWARPS * 32, NWARPS <= 12 ? 12 / NWARPS : 1)  // twelve warps per SM: at most 168 registers
paged_decode_fp8_partial_tma_kernel(const KernelParams p, const TmaParams tp,
                                    const __grid_constant__ CUtensorMap tmap_k,
                                    const __grid_constant__ CUtensorMap tmap_v) {
  constexpr int D = 128;
  constexpr uint32_t kTileBytes = kPage * D;  // 2 KiB
  constexpr uint32_t kStageBytes = 4 * kTileBytes;
  pdl_launch_dependents();
  const int dbg_slot = 1024 + blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);  // tuning builds only
  dbg_mark(dbg_slot, 0, threadIdx.x == 0);
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_v)) : "memory");
  }
  // Launched as a programmatic dependent of whatever precedes it in the stream: the CTA may
  // become resident while that kernel drains, but touches no memory before it has completed.
  // (Behind the dense prefix pass the wait is at the end instead: the two passes are independent.)
  // With early_metadata the caller vouches that seq_lens and block_table are not written by
  // that kernel: their reads below are then allowed to come first.
  if (p.slot_offset == 0 && !p.early_metadata) pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, i = lane >> 2, j = lane & 3;
  const int kv0 = kv_start_of(p, b);
  const int split_sz = split_size_of(p, kv0);
  const int lo = kv0 + split * split_sz;

  // Page ids of this warp's first 16 page pairs, one page per lane, fetched before the
  // sequence length is known (the block-table row is bt_cols wide, so this stays inside it).
  const int page_first = lo / kPage;
  auto my_page = [&](int pair, int u) { return page_first + (warp + pair * NWARPS) * 2 + u; };
  int ids_base = 0;
  int32_t ids = 0;
  {
    const int pg = my_page(lane >> 1, lane & 1);
    if (pg < p.bt_cols) ids = page_of(p.block_table, p.bt_stride_b, b, pg);
  }
  const int seq_len = p.seq_lens[b];
  const int hi = min(lo + split_sz, seq_len);
  // grouped decode: the grid was sized from the caller's bound on the suffixes; a request that
  // needs more splits than the grid has would lose its tail silently, so it is reported instead
  if (p.row_kv_start != nullptr && split == 0 && kvh == 0 && threadIdx.x == 0 &&
      seq_len - kv0 > (int)gridDim.x * split_sz)
    atomicExch(tp.status, kErrSuffixBound);
  // Behind the dense prefix pass (slot_offset > 0) this grid reads nothing of that pass, but it must
  // not COMPLETE before it: the merge kernel waits for this grid only.  One CTA that waits before
  // it exits is enough for that, and the others give their place on the SM to the next CTA.
  const bool waits_at_exit = p.slot_offset == 0 || (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
  if (lo >= hi) {
    if (waits_at_exit) pdl_wait();
    if (split == 0 && gridDim.x == 1 && p.direct_out) write_empty_rows<D>(p, b, kvh);
    return;
  }
  if (p.slot_offset == 0 && p.early_metadata) pdl_wait();
  dbg_mark(dbg_slot, 6, threadIdx.x == 0);  // sequence length known
  const int nsplits_seq = (seq_len - kv0 + split_sz - 1) / split_sz;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  // after the ring: mbarriers, then the small merge arrays; sm_o aliases the ring at the end
  const uint32_t bars = ring + NWARPS * NSTAGE * kStageBytes;
  float* sm_m = reinterpret_cast<float*>(ring_ptr + NWARPS * NSTAGE * kStageBytes + NWARPS * NSTAGE * 8);
  float* sm_l = sm_m + NWARPS * 16;
  float* sm_o = reinterpret_cast<float*>(ring_ptr);
  static_assert(NSTAGE * kStageBytes >= 16 * D * 4, "merge buffer must fit in the ring");

  const uint32_t my_ring = ring + warp * NSTAGE * kStageBytes;
  const uint32_t my_bars = bars + warp * NSTAGE * 8;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) mbar_init(my_bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies' completions see initialised barriers
  }
  __syncwarp();

  const int page_last = (hi - 1) / kPage;
  const int n_pairs_cta = (page_last - page_first + 2) / 2;
  const int n_pairs = (n_pairs_cta - warp + NWARPS - 1) / NWARPS;  // pairs warp, warp+NWARPS, ...

  auto issue = [&](int t, int32_t phys0, int32_t phys1) {  // lane 0 only
    const int s = t % NSTAGE;
    const uint32_t bar = my_bars + 8 * s;
    const uint32_t dst = my_ring + s * kStageBytes;
    const bool two = my_page(t, 1) <= page_last;
    mbar_expect_tx(bar, two ? kStageBytes : kStageBytes / 2);
    const int c1 = tp.head_is_dim1 ? kvh : 0;
    const int c2 = tp.head_is_dim1 ? 0 : kvh;
    if (p.kv_evict_first) {
      const uint64_t pol = l2_policy_evict_first();
      tma_load_tile(dst, &tmap_k, bar, c1, c2, phys0, pol);
      tma_load_tile(dst + 2 * kTileBytes, &tmap_v, bar, c1, c2, phys0, pol);
      if (two) {
        tma_load_tile(dst + kTileBytes, &tmap_k, bar, c1, c2, phys1, pol);
        tma_load_tile(dst + 3 * kTileBytes, &tmap_v, bar, c1, c2, phys1, pol);
      }
    } else {
      tma_load_tile(dst, &tmap_k, bar, c1, c2, phys0);
      tma_load_tile(dst + 2 * kTileBytes, &tmap_v, bar, c1, c2, phys0);
      if (two) {
        tma_load_tile(dst + kTileBytes, &tmap_k, bar, c1, c2, phys1);
        tma_load_tile(dst + 3 * kTileBytes, &tmap_v, bar, c1, c2, phys1);
      }
    }
  };
#pragma unroll
  for (int t = 0; t < NSTAGE; ++t) {
    const int32_t phys0 = __shfl_sync(0xffffffffu, ids, (2 * t) & 31);
    const int32_t phys1 = __shfl_sync(0xffffffffu, ids, (2 * t + 1) & 31);
    if (lane == 0 && t < n_pairs) issue(t, phys0, phys1);
  }
  dbg_mark(dbg_slot, 3, threadIdx.x == 0);  // first copies issued

  uint32_t qa[D / 16][4];
  load_q_frags<D, QBF16>(qa, p, b, kvh, i, j);
  const float ks = p.k_scale_ph ? __ldg(p.k_scale_ph + kvh) : p.k_scale;
  const float vs = p.v_scale_ph ? __ldg(p.v_scale_ph + kvh) : p.v_scale;
  const float scale_log2 = ks * p.sm_scale * kLog2e;

  WarpState<D> st;
#pragma unroll
  for (int m = 0; m < D / 8; ++m) st.o[m][0] = st.o[m][1] = st.o[m][2] = st.o[m][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

  // swizzled shared-memory offsets of this thread's fragments inside a tile
  uint32_t k_off[2][2], v_off[4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int l = 0; l < 2; ++l)
      k_off[nt][l] = (nt * 8 + rho(i)) * D + (((j + 4 * l) ^ rho(i)) << 4);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = v_row(j, r);
    v_off[r] = row * D + ((i ^ (row & 7)) << 4);
  }

  bool ok = true;
  int t = 0;
  for (; t < n_pairs; ++t) {
    const int s = t % NSTAGE;
    const uint32_t parity = (t / NSTAGE) & 1;
    if (!mbar_wait_bounded(my_bars + 8 * s, parity, tp.wait_limit_ns)) { ok = false; break; }
    if (t == 0) dbg_mark(dbg_slot, 4, threadIdx.x == 0);  // first pair arrived
    const uint32_t stage = my_ring + s * kStageBytes;
    const int tok0 = my_page(t, 0) * kPage;
    // the second page of the last pair may not exist: its (stale) bytes are masked like any
    // token beyond `hi`
    const bool edge = (tok0 < lo) | (tok0 + 2 * kPage > hi);
    float sc[4][4];
    uint32_t pa[2][4];
    {
      uint32_t k[4][2][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int l = 0; l < 2; ++l) {
          const uint4 x = lds_16(stage + (nt >> 1) * kTileBytes + k_off[nt & 1][l]);
          k[nt][l][0] = x.x; k[nt][l][1] = x.y; k[nt][l][2] = x.z; k[nt][l][3] = x.w;
        }
      qk_scores<D, 4>(sc, k, qa);
    }
    softmax_step<D, 4>(st, sc, pa, scale_log2, edge, tok0, lo, hi, j);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      uint32_t v[4][4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint4 x = lds_16(stage + (2 + u) * kTileBytes + v_off[r]);
        v[r][0] = x.x; v[r][1] = x.y; v[r][2] = x.z; v[r][3] = x.w;
      }
      pv_accumulate<D>(st, v, pa[u], edge, tok0 + u * kPage, lo, hi, j);
    }
    // Every byte this warp read from the stage has been consumed by an MMA above, so the
    // reads are complete: hand the stage back to TMA for the warp's pair t + NSTAGE.
    __syncwarp();
    const int tn = t + NSTAGE;
    if (tn < n_pairs) {
      if ((tn & 15) == 0) {  // next batch of 16 page pairs
        ids_base = tn;
        ids = 0;
        const int pg = my_page(tn + (lane >> 1), lane & 1);
        if (pg <= page_last) ids = page_of(p.block_table, p.bt_stride_b, b, pg);
      }
      const int32_t phys0 = __shfl_sync(0xffffffffu, ids, (2 * (tn - ids_base)) & 31);
      const int32_t phys1 = __shfl_sync(0xffffffffu, ids, (2 * (tn - ids_base) + 1) & 31);
      if (lane == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(tn, phys0, phys1);
      }
    }
  }
  dbg_mark(dbg_slot, 5, threadIdx.x == 0);  // pairs consumed
  if (!ok) {
    // Record the failure, then give this warp's copies still in flight a bounded chance to
    // land before the ring is reused by the merge below.
    if (lane == 0) {
      atomicExch(tp.status, kErrTmaTimeout);
      const int issued = min(n_pairs, t + NSTAGE);
      for (int u = t + 1; u < issued; ++u) mbar_wait_bounded(my_bars + 8 * (u % NSTAGE), (u / NSTAGE) & 1, tp.wait_limit_ns);
    }
    __syncwarp();
  }
  __syncthreads();  // every warp is done with its ring: sm_o may alias it
  cta_merge_and_store<D, QBF16, NWARPS>(st, p, b, kvh, split, nsplits_seq, vs, sm_m, sm_l, sm_o);
  dbg_mark(dbg_slot, 1, threadIdx.x == 0);
  // (see waits_at_exit; a no-op for an ordinary launch, which has waited before its first access)
  if (waits_at_exit) pdl_wait();
  dbg_mark(dbg_slot, 2, threadIdx.x == 0);
}

// LSE merge over the live splits of each (sequence, q head).  WPR = 1: one warp per row, four
// rows per CTA; WPR = 4 (few rows, many splits): the four warps of a CTA share one row, warp w
// taking splits w, w + 4, ..., and combine through shared memory.
// Same maths as _paged_split_kv_reduce (integrations/vllm/l20_paged_split_kv.py:459-488).
template <int D, bool QBF16, int WPR = 1>
__global__ void __launch_bounds__(128)
paged_decode_merge_kernel(const KernelParams p, int batch) {
  static_assert(WPR == 1 || WPR == 4, "one or four warps per row");
  pdl_launch_dependents();
  dbg_mark(4096 + blockIdx.x, 0, threadIdx.x == 0);
  const int warp = threadIdx.x >> 5;
  const int row = WPR == 1 ? blockIdx.x * 4 + warp : blockIdx.x;
  const int part = WPR == 1 ? 0 : warp;
  const int lane = threadIdx.x & 31;
  // This grid must not complete before the partial kernel has (the next kernel of the stream
  // would start while the partial kernel is still writing): warps with nothing to do leave at
  // once, but the last CTA of the grid always waits.
  const bool keeper = blockIdx.x == gridDim.x - 1;
  if (row >= batch * p.num_q_heads) {  // WPR == 1 only: whole warps, no barrier below
    if (keeper) pdl_wait();
    return;
  }
  const int b = row / p.num_q_heads, hq = row % p.num_q_heads;
  const int seq_len = p.seq_lens[b];
  const int kv0 = kv_start_of(p, b);
  const int live = seq_len - kv0;
  // slots in front of the splits: all slot_offset of them, or (grouped) those of this row's prefix
  const int pre = p.row_kv_start != nullptr ? (kv0 + 255) / 256 : p.slot_offset;
  const int skip = p.slot_offset - pre;  // unused slots between the row's prefix chunks and its splits
  const int split_sz = split_size_of(p, kv0);
  const int ns = (live > 0 ? (live + split_sz - 1) / split_sz : 0) + pre;
  constexpr int E = D / 32;  // elements per lane
  float acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  float big = -INFINITY, den = 0.f;
  if (ns == 1 && p.direct_out) {  // written by the partial kernel (with WPR == 4 the whole CTA returns)
    if (keeper) pdl_wait();
    return;
  }
  pdl_wait();  // the partial kernel's stores are complete and visible from here on
  dbg_mark(4096 + blockIdx.x, 1, threadIdx.x == 0);
  if (ns > 0) {
    const int64_t base = (int64_t)b * p.partial_stride_b + (int64_t)hq * p.partial_stride_h;
    // One pass with a running maximum; eight splits per round trip, their maxima, sums and data
    // requested together.
    for (int s0 = part; s0 < ns; s0 += 8 * WPR) {
      float mv[8], lv[8], xv[8][E];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool on = s0 + u * WPR < ns;
        const int k = on ? s0 + u * WPR : 0;  // (an idle lane re-reads the row's first live slot: finite data, weight 0)
        const int64_t pidx = base + (int64_t)(k < pre ? k : k + skip) * p.partial_stride_s;
        mv[u] = on ? p.partial_max[pidx] : -INFINITY;
        lv[u] = on ? p.partial_sum[pidx] : 0.f;
        if (p.partial_dtype == 0) {
          const float* src = reinterpret_cast<const float*>(p.partial_output) + pidx * D + lane * E;
          if constexpr (E == 4) {
            const float4 x = *reinterpret_cast<const float4*>(src);
            xv[u][0] = x.x; xv[u][1] = x.y; xv[u][2] = x.z; xv[u][3] = x.w;
          } else {
            const float2 x = *reinterpret_cast<const float2*>(src);
            xv[u][0] = x.x; xv[u][1] = x.y;
          }
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e) xv[u][e] = load_partial_elem(p.partial_output, p.partial_dtype, pidx * D + lane * E + e);
        }
      }
      float m_new = big;
#pragma unroll
      for (int u = 0; u < 8; ++u) m_new = fmaxf(m_new, mv[u]);
      const float keep = (big == -INFINITY) ? 0.f : expf(big - m_new);
      den *= keep;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] *= keep;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float c = (mv[u] == -INFINITY) ? 0.f : expf(mv[u] - m_new);
        den += lv[u] * c;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] += c * xv[u][e];
      }
      big = m_new;
    }
  }
  if constexpr (WPR == 4) {
    __shared__ float sh_acc[4][D];
    __shared__ float sh_m[4], sh_l[4];
#pragma unroll
    for (int e = 0; e < E; ++e) sh_acc[warp][lane * E + e] = acc[e];
    if (lane == 0) { sh_m[warp] = big; sh_l[warp] = den; }
    __syncthreads();
    if (warp != 0) return;
    const float m_all = fmaxf(fmaxf(sh_m[0], sh_m[1]), fmaxf(sh_m[2], sh_m[3]));
    den = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (sh_m[w] == -INFINITY) ? 0.f : expf(sh_m[w] - m_all);
      den += sh_l[w] * c;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] += c * sh_acc[w][lane * E + e];
    }
    big = m_all;
  }
  if (p.packed_output != nullptr) {
    float* dst = p.packed_output + (int64_t)row * (D + 2);
#pragma unroll
    for (int e = 0; e < E; ++e) dst[lane * E + e] = acc[e];
    if (lane == 0) { dst[D] = big; dst[D + 1] = den; }
    return;
  }
  dbg_mark(4096 + blockIdx.x, 2, threadIdx.x == 0);
  const float inv = ns > 0 ? 1.f / den : 0.f;
  const int64_t oidx = (int64_t)b * p.o_stride_b + (int64_t)hq * p.o_stride_h + lane * E;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float v = acc[e] * inv;
    if constexpr (QBF16) reinterpret_cast<__nv_bfloat16*>(p.output)[oidx + e] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(p.output)[oidx + e] = __float2half_rn(v);
  }
}

// Merge of packed partials [parts, rows, D+2] (o, m, l) -> output [rows, D]; one warp per row.
template <int D>
__global__ void __launch_bounds__(128)
merge_packed_kernel(const float* __restrict__ packed, int parts, int64_t rows, void* output,
                    int out_dtype) {
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  constexpr int E = D / 32;
  float big = -INFINITY;
  for (int s = lane; s < parts; s += 32) big = fmaxf(big, packed[((int64_t)s * rows + row) * (D + 2) + D]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
  float acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  float den = 0.f;
  for (int s = 0; s < parts; ++s) {
    const float* src = packed + ((int64_t)s * rows + row) * (D + 2);
    const float m = src[D];
    const float c = (m == -INFINITY) ? 0.f : expf(m - big);
    den += src[D + 1] * c;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] += c * src[lane * E + e];
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float v = acc[e] * inv;
    const int64_t idx = row * D + lane * E + e;
    if (out_dtype == 0) reinterpret_cast<float*>(output)[idx] = v;
    else if (out_dtype == 1) reinterpret_cast<__half*>(output)[idx] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(output)[idx] = __float2bfloat16_rn(v);
  }
}

constexpr int kErrPeerTimeout = 4;

// Receiving side of the KV-range exchange, one warp per row: the warp polls rank s's copy of the
// row in this rank's receive buffer until every word it needs carries this step's tag (the other
// GPUs' kernels store them; this GPU's own kernels have completed by then, the grid being their
// programmatic dependent), folds it into the running LSE merge and goes on to rank s + 1.  The
// wait is bounded in time: when it runs out the error word is set and the row is left alone.
// Either way the CTA that finishes last advances the count of completed steps.
template <int D>
__global__ void __launch_bounds__(128)
exchange_merge_kernel(const unsigned long long* __restrict__ recv, uint32_t* control, int world, int64_t rows,
                      void* output, int out_dtype, TmaParams tp) {
  static_assert(D == 128, "row layout");
  constexpr int kStampBase = 148 * 8 + 4096;  // rows of the stamp buffer (tuning builds only)
  mark_phase_at(tp, kStampBase + blockIdx.x, 0, threadIdx.x == 0);
  // The next kernel in the stream may be set up while this one waits for the other GPUs; whatever
  // it does before its own dependency wait touches nothing this grid reads or writes.
  pdl_launch_dependents();
  pdl_wait();  // this GPU's own rows are in place: from here on only other GPUs are waited for
  mark_phase_at(tp, kStampBase + blockIdx.x, 1, threadIdx.x == 0);
  const uint32_t step = __ldcg(control) + 1u;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row < rows) {
    const unsigned long long* base = recv + ((int64_t)(step & 1u) * world * rows + row) * kXchRow;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float big = -INFINITY, den = 0.f;
    bool complete = true;
    unsigned long long t0 = 0;
    for (int s = 0; s < world && complete; ++s) {
      const unsigned long long* src = base + (int64_t)s * rows * kXchRow;
      float4 x;
      float m, l;
      bool here = false;
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        bool ok = xch_load2(src + lane * 4, step, x.x, x.y);
        ok = xch_load2(src + lane * 4 + 2, step, x.z, x.w) && ok;
        ok = xch_load2(src + D, step, m, l) && ok;
        here = __all_sync(0xffffffffu, ok);
        if (here) break;
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (__any_sync(0xffffffffu, now - t0 > tp.wait_limit_ns)) break;
      }
      if (!here) { complete = false; break; }
      const float m_new = fmaxf(big, m);
      const float c_old = (big == -INFINITY) ? 0.f : expf(big - m_new);
      const float c = (m == -INFINITY) ? 0.f : expf(m - m_new);
      den = den * c_old + l * c;
      acc.x = acc.x * c_old + c * x.x; acc.y = acc.y * c_old + c * x.y;
      acc.z = acc.z * c_old + c * x.z; acc.w = acc.w * c_old + c * x.w;
      big = m_new;
    }
    if (complete) {
      mark_phase_at(tp, kStampBase + blockIdx.x, 2, threadIdx.x == 0);
      const float inv = den > 0.f ? 1.f / den : 0.f;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
      const int64_t idx = row * D + lane * 4;
      if (out_dtype == 0) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(output) + idx) = acc;
      } else if (out_dtype == 1) {
        const uint2 v = make_uint2(pack_f16x2(acc.x, acc.y), pack_f16x2(acc.z, acc.w));
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(output) + idx) = v;
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        const uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(output) + idx) = v;
      }
    } else if (lane == 0) {
      atomicExch(tp.status, kErrPeerTimeout);
    }
  }
  // every warp of the grid has read the step count above; the last CTA to get here advances it
  __syncthreads();
  mark_phase_at(tp, kStampBase + blockIdx.x, 3, threadIdx.x == 0);
  if (threadIdx.x == 0) {
    if (atomicAdd(control + 1, 1u) == gridDim.x - 1) {
      atomicExch(control + 1, 0u);
      atomicAdd(control, 1u);
    }
  }
}

__global__ void resolve_slots_kernel(const int32_t* __restrict__ block_table, int64_t bt_stride_b,
                                     const int32_t* __restrict__ seq_lens, int max_seq_len,
                                     int64_t* __restrict__ slots) {
  const int b = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= max_seq_len) return;
  int64_t slot = -1;
  if (t < seq_lens[b]) slot = (int64_t)page_of(block_table, bt_stride_b, b, t / kPage) * kPage + t % kPage;
  slots[(int64_t)b * max_seq_len + t] = slot;
}

}  // namespace pfd
