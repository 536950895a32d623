// The producer step in front of decode attention: rotary embedding of the new tokens' Q and K
// (in place), then K and V written into the paged cache at the slots the engine assigned --
// into fp16 / bf16 caches as they are, into FP8-e4m3 caches divided by a per-(layer, kv head)
// scale.  Same call as the reference's fused operator (integrations/vllm/l20_rope_kv.py:256-328,
// kernels :26-253), which refuses quantised caches (:273-274).
//
// One CTA per token.  The arithmetic is written so that a CPU restatement in torch reproduces
// it bit for bit: products and the sum of the rotation are rounded separately (no fused
// multiply-add), the rotated value is rounded to the model's 16-bit type first (that is what
// stays in `key` / `query`), and the FP8 value is that rounded number divided by the scale in
// fp32, saturated to +-448 and rounded to nearest even.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace pfd {

struct RopeParams {
  void* query;        // [T, Hq, D], rotated in place
  void* key;          // [T, Hkv, D], rotated in place
  const void* value;  // [T, Hkv, D]
  const int64_t* positions;     // [T]
  const void* cos_sin_cache;    // [max_position, rotary_dim]: cos of the rotary_dim / 2 frequencies, then sin
  const int64_t* slot_mapping;  // [T]: block * block_size + offset, negative = do not store
  void* key_cache;              // logical [blocks, block_size, Hkv, D]
  void* value_cache;
  const float* k_scale_ph;  // FP8 caches: per kv head, or the scalars below
  const float* v_scale_ph;
  float k_scale, v_scale;
  int64_t q_stride_t, q_stride_h, k_stride_t, k_stride_h, v_stride_t, v_stride_h;  // elements
  int64_t kc_stride_block, kc_stride_token, kc_stride_head;                          // elements of the cache
  int64_t vc_stride_block, vc_stride_token, vc_stride_head;
  int64_t cs_stride;  // elements between rows of cos_sin_cache
  int32_t num_tokens, num_q_heads, num_kv_heads, head_dim, rotary_dim, block_size;
  int32_t is_neox;       // 1: pairs (i, i + rotary_dim / 2); 0: pairs (2i, 2i + 1)
  int32_t cos_sin_f32;   // 1: cos_sin_cache is float32, 0: it has the query's type
  int32_t cache_fp8;     // 1: e4m3 caches, 0: caches of the query's type
};

template <bool BF16>
__device__ __forceinline__ float load16(const void* p, int64_t i) {
  if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  else return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
template <bool BF16>
__device__ __forceinline__ float round16(float x) {  // x rounded to the 16-bit type, as a float
  if constexpr (BF16) return __bfloat162float(__float2bfloat16_rn(x));
  else return __half2float(__float2half_rn(x));
}
template <bool BF16>
__device__ __forceinline__ void store16(void* p, int64_t i, float x) {
  if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
}
__device__ __forceinline__ uint8_t to_e4m3(float x, float scale) {
  // x / scale in fp32 (IEEE division), saturate-to-finite, round to nearest even
  const float y = __fdiv_rn(x, scale);
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(y));
  return static_cast<uint8_t>(r & 0xffu);
}

template <bool BF16>
__global__ void __launch_bounds__(256) rope_quant_append_kernel(const RopeParams p) {
  // lets a kernel launched behind this one as a programmatic dependent become resident while this
  // one runs (the decode kernels, which wait for its completion before they touch what it writes)
  asm volatile("griddepcontrol.launch_dependents;");
  const int t = blockIdx.x;
  const int64_t pos = p.positions[t];
  const int64_t slot = p.slot_mapping[t];
  const int half = p.rotary_dim / 2;
  const int D = p.head_dim;
  const auto cs = [&](int f, bool sine) -> float {
    const int64_t i = pos * p.cs_stride + (sine ? half : 0) + f;
    return p.cos_sin_f32 ? reinterpret_cast<const float*>(p.cos_sin_cache)[i] : load16<BF16>(p.cos_sin_cache, i);
  };
  const int64_t block = slot >= 0 ? slot / p.block_size : 0;
  const int64_t offset = slot >= 0 ? slot % p.block_size : 0;

  // rotation pairs of the Q heads and of the K heads: one (head, frequency) per thread-iteration
  const int heads = p.num_q_heads + p.num_kv_heads;
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int head = e / half, f = e % half;
    const bool is_q = head < p.num_q_heads;
    const int h = is_q ? head : head - p.num_q_heads;
    void* base = is_q ? p.query : p.key;
    const int64_t row = is_q ? (int64_t)t * p.q_stride_t + (int64_t)h * p.q_stride_h
                             : (int64_t)t * p.k_stride_t + (int64_t)h * p.k_stride_h;
    const int d1 = p.is_neox ? f : 2 * f, d2 = p.is_neox ? f + half : 2 * f + 1;
    const float x1 = load16<BF16>(base, row + d1), x2 = load16<BF16>(base, row + d2);
    const float c = cs(f, false), s = cs(f, true);
    const float y1 = round16<BF16>(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
    const float y2 = round16<BF16>(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
    store16<BF16>(base, row + d1, y1);
    store16<BF16>(base, row + d2, y2);
    if (!is_q && slot >= 0) {
      const int64_t dst = block * p.kc_stride_block + offset * p.kc_stride_token + (int64_t)h * p.kc_stride_head;
      if (p.cache_fp8) {
        const float sc = p.k_scale_ph ? p.k_scale_ph[h] : p.k_scale;
        reinterpret_cast<uint8_t*>(p.key_cache)[dst + d1] = to_e4m3(y1, sc);
        reinterpret_cast<uint8_t*>(p.key_cache)[dst + d2] = to_e4m3(y2, sc);
      } else {
        store16<BF16>(p.key_cache, dst + d1, y1);
        store16<BF16>(p.key_cache, dst + d2, y2);
      }
    }
  }
  if (slot < 0) return;
  // the part of K behind rotary_dim (not rotated), and V
  for (int e = threadIdx.x; e < p.num_kv_heads * D; e += blockDim.x) {
    const int h = e / D, d = e % D;
    const int64_t kdst = block * p.kc_stride_block + offset * p.kc_stride_token + (int64_t)h * p.kc_stride_head + d;
    const int64_t vdst = block * p.vc_stride_block + offset * p.vc_stride_token + (int64_t)h * p.vc_stride_head + d;
    const float v = load16<BF16>(p.value, (int64_t)t * p.v_stride_t + (int64_t)h * p.v_stride_h + d);
    if (p.cache_fp8) {
      reinterpret_cast<uint8_t*>(p.value_cache)[vdst] = to_e4m3(v, p.v_scale_ph ? p.v_scale_ph[h] : p.v_scale);
    } else {
      store16<BF16>(p.value_cache, vdst, v);
    }
    if (d >= p.rotary_dim) {
      const float k = load16<BF16>(p.key, (int64_t)t * p.k_stride_t + (int64_t)h * p.k_stride_h + d);
      if (p.cache_fp8) reinterpret_cast<uint8_t*>(p.key_cache)[kdst] = to_e4m3(k, p.k_scale_ph ? p.k_scale_ph[h] : p.k_scale);
      else store16<BF16>(p.key_cache, kdst, k);
    }
  }
}

// ---- the common case, vectorised -------------------------------------------------------------
// NeoX pairing over the whole head (rotary_dim == head_dim), head_dim a multiple of 16, every
// row 16-byte aligned.  A task is eight consecutive frequencies of one head -- two 16-byte loads
// of the head (elements f .. f + 7 and f + half .. f + half + 7), the eight cosines and sines,
// two 16-byte stores back and, for a K head, two stores into the cache (8 bytes each as e4m3,
// converted two at a time) -- or eight consecutive elements of one V head.  The tasks of a token
// are dealt to the threads of its CTA.  Element by element the arithmetic is that of the kernel
// above, so the results are the same bits.
struct Vec8 {
  float v[8];
};
template <bool BF16>
__device__ __forceinline__ Vec8 load8(const void* base, int64_t i) {  // 8 consecutive 16-bit elements, 16-byte aligned
  const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + i);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  Vec8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if constexpr (BF16) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[k]);
      r.v[2 * k] = __bfloat162float(h.x); r.v[2 * k + 1] = __bfloat162float(h.y);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[k]);
      r.v[2 * k] = __half2float(h.x); r.v[2 * k + 1] = __half2float(h.y);
    }
  }
  return r;
}
template <bool BF16>
__device__ __forceinline__ void store8(void* base, int64_t i, const Vec8& x) {  // rounds to the 16-bit type
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if constexpr (BF16) {
      __nv_bfloat162 h;
      h.x = __float2bfloat16_rn(x.v[2 * k]); h.y = __float2bfloat16_rn(x.v[2 * k + 1]);
      w[k] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __half2 h;
      h.x = __float2half_rn(x.v[2 * k]); h.y = __float2half_rn(x.v[2 * k + 1]);
      w[k] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + i) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store8_e4m3(void* cache, int64_t i, const Vec8& x, float scale) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint16_t r;  // the first operand lands in the upper byte
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(__fdiv_rn(x.v[2 * k + 1], scale)), "f"(__fdiv_rn(x.v[2 * k], scale)));
    w[k >> 1] |= (uint32_t)r << (16 * (k & 1));
  }
  *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(cache) + i) = make_uint2(w[0], w[1]);
}

template <bool BF16>
__global__ void __launch_bounds__(256) rope_quant_append_vec_kernel(const RopeParams p) {
  // lets a kernel launched behind this one as a programmatic dependent become resident while this
  // one runs (the decode kernels, which wait for its completion before they touch what it writes)
  asm volatile("griddepcontrol.launch_dependents;");
  const int t = blockIdx.x;
  const int64_t pos = p.positions[t];
  const int64_t slot = p.slot_mapping[t];
  const int D = p.head_dim, half = D / 2;
  const int per_head = half / 8;                       // rotation tasks per head
  const int heads = p.num_q_heads + p.num_kv_heads;
  const int n_rot = heads * per_head;
  const int n_val = slot >= 0 ? p.num_kv_heads * (D / 8) : 0;
  const int64_t block = slot >= 0 ? slot / p.block_size : 0;
  const int64_t offset = slot >= 0 ? slot % p.block_size : 0;
  for (int e = threadIdx.x; e < n_rot + n_val; e += blockDim.x) {
    if (e < n_rot) {
      const int head = e / per_head, f = (e % per_head) * 8;
      const bool is_q = head < p.num_q_heads;
      const int h = is_q ? head : head - p.num_q_heads;
      void* base = is_q ? p.query : p.key;
      const int64_t row = is_q ? (int64_t)t * p.q_stride_t + (int64_t)h * p.q_stride_h
                               : (int64_t)t * p.k_stride_t + (int64_t)h * p.k_stride_h;
      const Vec8 x1 = load8<BF16>(base, row + f), x2 = load8<BF16>(base, row + f + half);
      Vec8 c, s;
      if (p.cos_sin_f32) {
        const float4* cp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.cos_sin_cache) + pos * p.cs_stride + f);
        const float4* sp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.cos_sin_cache) + pos * p.cs_stride + half + f);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c = Vec8{{c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}};
        s = Vec8{{s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w}};
      } else {
        c = load8<BF16>(p.cos_sin_cache, pos * p.cs_stride + f);
        s = load8<BF16>(p.cos_sin_cache, pos * p.cs_stride + half + f);
      }
      Vec8 y1, y2;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        y1.v[k] = round16<BF16>(__fsub_rn(__fmul_rn(x1.v[k], c.v[k]), __fmul_rn(x2.v[k], s.v[k])));
        y2.v[k] = round16<BF16>(__fadd_rn(__fmul_rn(x2.v[k], c.v[k]), __fmul_rn(x1.v[k], s.v[k])));
      }
      store8<BF16>(base, row + f, y1);
      store8<BF16>(base, row + f + half, y2);
      if (!is_q && slot >= 0) {
        const int64_t dst = block * p.kc_stride_block + offset * p.kc_stride_token + (int64_t)h * p.kc_stride_head;
        if (p.cache_fp8) {
          const float sc = p.k_scale_ph ? p.k_scale_ph[h] : p.k_scale;
          store8_e4m3(p.key_cache, dst + f, y1, sc);
          store8_e4m3(p.key_cache, dst + f + half, y2, sc);
        } else {
          store8<BF16>(p.key_cache, dst + f, y1);
          store8<BF16>(p.key_cache, dst + f + half, y2);
        }
      }
    } else {
      const int v = e - n_rot;
      const int h = v / (D / 8), d = (v % (D / 8)) * 8;
      const Vec8 x = load8<BF16>(p.value, (int64_t)t * p.v_stride_t + (int64_t)h * p.v_stride_h + d);
      const int64_t dst = block * p.vc_stride_block + offset * p.vc_stride_token + (int64_t)h * p.vc_stride_head + d;
      if (p.cache_fp8) store8_e4m3(p.value_cache, dst, x, p.v_scale_ph ? p.v_scale_ph[h] : p.v_scale);
      else store8<BF16>(p.value_cache, dst, x);
    }
  }
}

}  // namespace pfd
