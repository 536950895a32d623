// PyTorch dispatcher surface of the B200 paged FP8 decode operator.
//
// Keeps the reference project's operator schema so that existing callers keep working:
//   TORCH_LIBRARY(l20_stack) "paged_decode_fp8_e4m3_split_out(...)"
//       integrations/vllm/cuda/l20_paged_decode.cpp:128-135 (schema), :138-143 (CUDA impl),
//       :153-155 (pybind export of the same launcher)
// and adds "paged_decode_fp8_e4m3_split_out_v2" (per-kv-head scale tensors, explicit softmax
// scale, kv_start, optional packed (o, m, l) output, PFD_FLAG_* bits, an optional plan),
// "plan_decode", "group_shared_prefixes", "merge_packed_partials" and "resolve_slots".  Every op only unpacks tensors
// into the C ABI of libpaged_fp8_decode.so
// (include/paged_fp8_decode.h); there is no computation here and no fallback.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "paged_fp8_decode.h"

namespace {

int32_t dtype_code(at::ScalarType t, const char* what) {
  if (t == at::kFloat) return PFD_DTYPE_F32;
  if (t == at::kHalf) return PFD_DTYPE_F16;
  if (t == at::kBFloat16) return PFD_DTYPE_BF16;
  TORCH_CHECK(false, what, " must be float32, float16 or bfloat16");
  return -1;
}

void run_decode(const at::Tensor& query, const at::Tensor& key_cache, const at::Tensor& value_cache,
                const at::Tensor& block_table, const at::Tensor& seq_lens,
                const c10::optional<at::Tensor>& partial_output,
                const c10::optional<at::Tensor>& partial_max,
                const c10::optional<at::Tensor>& partial_sum, const c10::optional<at::Tensor>& output,
                const c10::optional<at::Tensor>& packed_output, double k_scale, double v_scale,
                const c10::optional<at::Tensor>& k_scale_ph, const c10::optional<at::Tensor>& v_scale_ph,
                double sm_scale, int64_t max_seq_len, int64_t split_size, int64_t kv_start,
                int64_t flags, const c10::optional<at::Tensor>& plan = c10::nullopt,
                int64_t prefix_len = 0, bool kv16 = false,
                const c10::optional<at::Tensor>& page_indptr = c10::nullopt, bool plan_only = false,
                const c10::optional<at::Tensor>& groups = c10::nullopt, int64_t max_groups = 0,
                int64_t max_prefix_len = 0, int64_t max_suffix_len = 0) {
  TORCH_CHECK(query.is_cuda(), "query must be CUDA");
  TORCH_CHECK(query.scalar_type() == at::kHalf || query.scalar_type() == at::kBFloat16,
              "query must be FP16 or BF16");
  if (kv16) {
    TORCH_CHECK(key_cache.scalar_type() == query.scalar_type() && value_cache.scalar_type() == query.scalar_type(),
                "K/V cache must have the query's dtype");
  } else {
    TORCH_CHECK(key_cache.scalar_type() == at::kFloat8_e4m3fn &&
                    value_cache.scalar_type() == at::kFloat8_e4m3fn,
                "K/V cache must be torch.float8_e4m3fn");
  }
  TORCH_CHECK(query.dim() == 3 && query.stride(2) == 1, "invalid query");
  TORCH_CHECK(key_cache.dim() == 4 && key_cache.size(3) == query.size(2) && key_cache.stride(3) == 1 &&
                  value_cache.dim() == 4 && value_cache.stride(3) == 1,
              "NHD cache only");
  TORCH_CHECK(key_cache.sizes() == value_cache.sizes(), "K/V cache mismatch");
  TORCH_CHECK(key_cache.is_cuda() && value_cache.is_cuda() && block_table.is_cuda() && seq_lens.is_cuda(),
              "all operands must be CUDA");
  if (page_indptr.has_value()) {  // block_table is the flat list of page ids the indptr indexes
    TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 1 && block_table.is_contiguous(),
                "int32 page indices");
    TORCH_CHECK(page_indptr->is_cuda() && page_indptr->scalar_type() == at::kInt && page_indptr->is_contiguous() &&
                    page_indptr->numel() == query.size(0) + 1,
                "int32 page indptr with batch + 1 entries");
  } else {
    TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 2 &&
                    block_table.stride(1) == 1 && block_table.size(0) == query.size(0),
                "int32 block table");
  }
  TORCH_CHECK(seq_lens.scalar_type() == at::kInt && seq_lens.is_contiguous() &&
                  seq_lens.numel() == query.size(0),
              "int32 sequence lengths");
  TORCH_CHECK(split_size >= 16 && split_size % 16 == 0, "split_size must be a multiple of 16");
  TORCH_CHECK(key_cache.size(2) > 0 && query.size(1) % key_cache.size(2) == 0,
              "Q heads must be divisible by KV heads");
  TORCH_CHECK(max_seq_len >= 0 && (page_indptr.has_value() ||
                                   max_seq_len <= block_table.size(1) * key_cache.size(1)),
              "max_seq_len exceeds the block table");

  pfd_decode_args a{};
  a.struct_size = sizeof(a);
  a.flags = static_cast<uint32_t>(flags);
  a.batch = static_cast<int32_t>(query.size(0));
  a.num_q_heads = static_cast<int32_t>(query.size(1));
  a.num_kv_heads = static_cast<int32_t>(key_cache.size(2));
  a.head_dim = static_cast<int32_t>(query.size(2));
  a.page_size = static_cast<int32_t>(key_cache.size(1));
  a.max_seq_len = static_cast<int32_t>(max_seq_len);
  a.split_size = static_cast<int32_t>(split_size);
  a.kv_start = static_cast<int32_t>(kv_start);
  a.query_dtype = dtype_code(query.scalar_type(), "query");
  a.sm_scale = static_cast<float>(sm_scale);
  a.k_scale = static_cast<float>(k_scale);
  a.v_scale = static_cast<float>(v_scale);
  a.query = query.data_ptr();
  a.q_stride_b = query.stride(0);
  a.q_stride_h = query.stride(1);
  a.key_cache = key_cache.data_ptr();
  a.value_cache = value_cache.data_ptr();
  a.num_pages = key_cache.size(0);
  a.k_stride_page = key_cache.stride(0);
  a.k_stride_token = key_cache.stride(1);
  a.k_stride_head = key_cache.stride(2);
  a.v_stride_page = value_cache.stride(0);
  a.v_stride_token = value_cache.stride(1);
  a.v_stride_head = value_cache.stride(2);
  a.block_table = block_table.data_ptr<int32_t>();
  a.bt_stride_b = page_indptr.has_value() ? 0 : block_table.stride(0);
  if (page_indptr.has_value()) a.page_indptr = page_indptr->data_ptr<int32_t>();
  a.seq_lens = seq_lens.data_ptr<int32_t>();
  if (k_scale_ph.has_value()) {
    TORCH_CHECK(k_scale_ph->is_cuda() && k_scale_ph->scalar_type() == at::kFloat &&
                    k_scale_ph->is_contiguous() && k_scale_ph->numel() == key_cache.size(2),
                "k_scale must be a float32 CUDA tensor with one entry per KV head");
    a.k_scale_per_head = k_scale_ph->data_ptr<float>();
  }
  if (v_scale_ph.has_value()) {
    TORCH_CHECK(v_scale_ph->is_cuda() && v_scale_ph->scalar_type() == at::kFloat &&
                    v_scale_ph->is_contiguous() && v_scale_ph->numel() == key_cache.size(2),
                "v_scale must be a float32 CUDA tensor with one entry per KV head");
    a.v_scale_per_head = v_scale_ph->data_ptr<float>();
  }
  if (partial_output.has_value()) {
    const at::Tensor& po = *partial_output;
    TORCH_CHECK(partial_max.has_value() && partial_sum.has_value(),
                "partial output workspace has wrong shape");
    TORCH_CHECK(po.is_cuda() && po.dim() == 4 && po.size(0) >= query.size(0) &&
                    po.size(1) == query.size(1) && po.size(3) == query.size(2) && po.is_contiguous(),
                "partial output workspace has wrong shape");
    TORCH_CHECK(partial_max->scalar_type() == at::kFloat && partial_sum->scalar_type() == at::kFloat &&
                    partial_max->is_contiguous() && partial_sum->is_contiguous() &&
                    partial_max->dim() == 3 && partial_max->sizes() == partial_sum->sizes() &&
                    partial_max->size(0) == po.size(0) && partial_max->size(1) == po.size(1) &&
                    partial_max->size(2) == po.size(2),
                "partial max/sum workspace has wrong shape");
    a.partial_dtype = dtype_code(po.scalar_type(), "partial_output");
    a.partial_output = po.data_ptr();
    a.partial_max = partial_max->data_ptr<float>();
    a.partial_sum = partial_sum->data_ptr<float>();
    a.partial_stride_b = partial_max->stride(0);
    a.partial_stride_h = partial_max->stride(1);
    a.partial_stride_s = partial_max->stride(2);
    a.workspace_splits = static_cast<int32_t>(po.size(2));
  }
  if (output.has_value()) {
    TORCH_CHECK(output->is_cuda() && output->scalar_type() == query.scalar_type() &&
                    output->sizes() == query.sizes() && output->stride(2) == 1,
                "output must match query");
    a.output = output->data_ptr();
    a.o_stride_b = output->stride(0);
    a.o_stride_h = output->stride(1);
  }
  if (packed_output.has_value()) {
    TORCH_CHECK(packed_output->is_cuda() && packed_output->scalar_type() == at::kFloat &&
                    packed_output->is_contiguous() && packed_output->dim() == 3 &&
                    packed_output->size(0) == query.size(0) && packed_output->size(1) == query.size(1) &&
                    packed_output->size(2) == query.size(2) + 2,
                "packed_output must be float32 [B, Hq, D + 2]");
    a.packed_output = packed_output->data_ptr<float>();
  }
  if (plan.has_value()) {
    TORCH_CHECK(plan->is_cuda() && plan->scalar_type() == at::kInt && plan->is_contiguous(),
                "plan must be a contiguous int32 CUDA tensor");
    a.plan = plan->data_ptr<int32_t>();
  }
  const at::cuda::CUDAGuard guard(query.device());
  a.stream = at::cuda::getCurrentCUDAStream().stream();
  if (plan_only) {
    TORCH_CHECK(plan.has_value(), "plan_decode needs a plan buffer");
    TORCH_CHECK(pfd_plan_decode(&a, kv16 ? 2 : 1, a.plan, plan->numel() * 4) == PFD_OK, pfd_last_error());
    return;
  }
  if (groups.has_value()) {
    TORCH_CHECK(groups->is_cuda() && groups->scalar_type() == at::kInt && groups->is_contiguous() &&
                    groups->numel() * 4 >= pfd_prefix_groups_bytes(a.batch, static_cast<int32_t>(max_groups)),
                "groups must be the int32 CUDA buffer group_shared_prefixes filled for this batch and max_groups");
    TORCH_CHECK(pfd_shared_prefix_decode_grouped_fp8_e4m3(&a, groups->data_ptr<int32_t>(), static_cast<int32_t>(max_groups),
                                                          static_cast<int32_t>(max_prefix_len),
                                                          static_cast<int32_t>(max_suffix_len)) == PFD_OK,
                pfd_last_error());
    return;
  }
  const int rc = kv16             ? pfd_paged_decode_kv16_split_out(&a)
                 : prefix_len > 0 ? pfd_shared_prefix_decode_fp8_e4m3(&a, static_cast<int32_t>(prefix_len))
                                  : pfd_paged_decode_fp8_e4m3_split_out(&a);
  TORCH_CHECK(rc == PFD_OK, pfd_last_error());
}

// Same argument list as the reference dispatch function
// (integrations/vllm/cuda/l20_paged_decode.cpp:89-118).
at::Tensor paged_decode_fp8_e4m3_split_out(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                           at::Tensor block_table, at::Tensor seq_lens,
                                           at::Tensor partial_output, at::Tensor partial_max,
                                           at::Tensor partial_sum, at::Tensor output, double k_scale,
                                           double v_scale, int64_t max_seq_len, int64_t split_size) {
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max,
             partial_sum, output, c10::nullopt, k_scale, v_scale, c10::nullopt, c10::nullopt, 0.0,
             max_seq_len, split_size, 0, 0);
  return output;
}

// The non-quantised sibling, same argument list as the reference dispatch function
// (integrations/vllm/cuda/l20_paged_decode.cpp:60-87; schema :121-127): caches in the query's dtype.
at::Tensor paged_decode_split_out(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                  at::Tensor block_table, at::Tensor seq_lens, at::Tensor partial_output,
                                  at::Tensor partial_max, at::Tensor partial_sum, at::Tensor output,
                                  int64_t max_seq_len, int64_t split_size) {
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max,
             partial_sum, output, c10::nullopt, 1.0, 1.0, c10::nullopt, c10::nullopt, 0.0,
             max_seq_len, split_size, 0, 0, c10::nullopt, 0, /*kv16=*/true);
  return output;
}

// Superset of the above: PFD_FLAG_* bits and an optional plan (pfd_plan_decode).
void paged_decode_split_out_v2(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                               at::Tensor block_table, at::Tensor seq_lens, at::Tensor partial_output,
                               at::Tensor partial_max, at::Tensor partial_sum, at::Tensor output,
                               int64_t max_seq_len, int64_t split_size, int64_t flags,
                               c10::optional<at::Tensor> plan) {
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max,
             partial_sum, output, c10::nullopt, 1.0, 1.0, c10::nullopt, c10::nullopt, 0.0,
             max_seq_len, split_size, 0, flags, plan, 0, /*kv16=*/true);
}

// The same with FlashInfer's page addressing (indptr [B + 1], indices): argument list of
// l20_paged_decode_split_indices_out_cuda (integrations/vllm/cuda/l20_paged_decode.cu:600-612).
void paged_decode_split_indices_out(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                    at::Tensor page_indptr, at::Tensor page_indices, at::Tensor seq_lens,
                                    at::Tensor partial_output, at::Tensor partial_max, at::Tensor partial_sum,
                                    at::Tensor output, int64_t max_seq_len, int64_t split_size) {
  run_decode(query, key_cache, value_cache, page_indices, seq_lens, partial_output, partial_max,
             partial_sum, output, c10::nullopt, 1.0, 1.0, c10::nullopt, c10::nullopt, 0.0,
             max_seq_len, split_size, 0, 0, c10::nullopt, 0, /*kv16=*/true, page_indptr);
}

void paged_decode_split_out_void(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                 at::Tensor block_table, at::Tensor seq_lens, at::Tensor partial_output,
                                 at::Tensor partial_max, at::Tensor partial_sum, at::Tensor output,
                                 int64_t max_seq_len, int64_t split_size) {
  paged_decode_split_out(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max,
                         partial_sum, output, max_seq_len, split_size);
}

void paged_decode_fp8_e4m3_split_out_void(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                          at::Tensor block_table, at::Tensor seq_lens,
                                          at::Tensor partial_output, at::Tensor partial_max,
                                          at::Tensor partial_sum, at::Tensor output, double k_scale,
                                          double v_scale, int64_t max_seq_len, int64_t split_size) {
  paged_decode_fp8_e4m3_split_out(query, key_cache, value_cache, block_table, seq_lens, partial_output,
                                  partial_max, partial_sum, output, k_scale, v_scale, max_seq_len,
                                  split_size);
}

void paged_decode_fp8_e4m3_split_out_v2(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                        at::Tensor block_table, at::Tensor seq_lens,
                                        c10::optional<at::Tensor> partial_output,
                                        c10::optional<at::Tensor> partial_max,
                                        c10::optional<at::Tensor> partial_sum,
                                        c10::optional<at::Tensor> output,
                                        c10::optional<at::Tensor> packed_output, at::Tensor k_scale,
                                        at::Tensor v_scale, double sm_scale, int64_t max_seq_len,
                                        int64_t split_size, int64_t kv_start, int64_t flags,
                                        c10::optional<at::Tensor> plan) {
  TORCH_CHECK(output.has_value() || packed_output.has_value(), "no output given");
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max,
             partial_sum, output, packed_output, 1.0, 1.0, k_scale, v_scale, sm_scale, max_seq_len,
             split_size, kv_start, flags, plan);
}

// The work split of a model step's decode calls (pfd_plan_decode), written into `plan`; the
// caches are passed for their geometry only.  plan.numel() * 4 >= plan_bytes(batch, kv heads).
void plan_decode(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache, at::Tensor block_table,
                 at::Tensor seq_lens, at::Tensor partial_output, at::Tensor partial_max, at::Tensor partial_sum,
                 at::Tensor plan, int64_t max_seq_len, int64_t split_size, int64_t kv_start) {
  const bool kv16 = key_cache.scalar_type() == query.scalar_type();
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum,
             c10::nullopt, c10::nullopt, 1.0, 1.0, c10::nullopt, c10::nullopt, 0.0, max_seq_len, split_size,
             kv_start, 0, plan, 0, kv16, c10::nullopt, /*plan_only=*/true);
}

int64_t plan_bytes(int64_t batch, int64_t num_kv_heads) {
  const int64_t n = pfd_plan_bytes(static_cast<int32_t>(batch), static_cast<int32_t>(num_kv_heads));
  TORCH_CHECK(n >= 0, pfd_last_error());
  return n;
}

// Decode step of a batch whose requests all share the first prefix_len tokens' pages: dense
// tcgen05 prefix pass + split-KV suffix pass + merge (pfd_shared_prefix_decode_fp8_e4m3).
void shared_prefix_decode_fp8_e4m3(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                   at::Tensor block_table, at::Tensor seq_lens, at::Tensor partial_output,
                                   at::Tensor partial_max, at::Tensor partial_sum, at::Tensor output,
                                   at::Tensor k_scale, at::Tensor v_scale, double sm_scale,
                                   int64_t max_seq_len, int64_t split_size, int64_t prefix_len) {
  TORCH_CHECK(prefix_len > 0, "prefix_len must be positive");
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum,
             output, c10::nullopt, 1.0, 1.0, k_scale, v_scale, sm_scale, max_seq_len, split_size, 0, 0,
             c10::nullopt, prefix_len);
}

void shared_prefix_decode_grouped_fp8_e4m3(at::Tensor query, at::Tensor key_cache, at::Tensor value_cache,
                                           at::Tensor block_table, at::Tensor seq_lens, at::Tensor partial_output,
                                           at::Tensor partial_max, at::Tensor partial_sum, at::Tensor output,
                                           at::Tensor k_scale, at::Tensor v_scale, double sm_scale,
                                           int64_t max_seq_len, int64_t split_size, at::Tensor groups,
                                           int64_t max_groups, int64_t max_prefix_len, int64_t max_suffix_len,
                                           bool all_in_groups) {
  run_decode(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum,
             output, c10::nullopt, 1.0, 1.0, k_scale, v_scale, sm_scale, max_seq_len, split_size, 0,
             all_in_groups ? PFD_FLAG_ALL_IN_GROUPS : 0, c10::nullopt, 0, false, c10::nullopt, false, groups, max_groups,
             max_prefix_len, max_suffix_len);
}

// Rotary embedding of the new tokens' query and key (in place) + append of key / value to the
// paged cache; argument list of the reference's l20_rope_and_cache
// (integrations/vllm/l20_rope_kv.py:256-266) plus the scales an FP8 cache needs.
void rope_and_cache(at::Tensor query, at::Tensor key, at::Tensor value, at::Tensor positions,
                    at::Tensor cos_sin_cache, bool is_neox, at::Tensor key_cache, at::Tensor value_cache,
                    at::Tensor slot_mapping, c10::optional<at::Tensor> k_scale, c10::optional<at::Tensor> v_scale) {
  TORCH_CHECK(query.is_cuda() && (query.scalar_type() == at::kHalf || query.scalar_type() == at::kBFloat16),
              "l20_rope_and_cache supports FP16 and BF16");
  TORCH_CHECK(key.scalar_type() == query.scalar_type() && value.scalar_type() == query.scalar_type(),
              "Q, K, and V must use the same dtype");
  TORCH_CHECK(query.dim() == 3 && key.dim() == 3 && value.dim() == 3, "Q, K, and V must be [tokens, heads, head_dim]");
  TORCH_CHECK(key.sizes() == value.sizes() && query.size(0) == key.size(0) && query.size(2) == key.size(2),
              "Q, K, and V shapes are incompatible");
  TORCH_CHECK(query.stride(2) == 1 && key.stride(2) == 1 && value.stride(2) == 1, "head_dim must be contiguous");
  const bool fp8 = key_cache.scalar_type() == at::kFloat8_e4m3fn || key_cache.scalar_type() == at::kByte;
  TORCH_CHECK(fp8 || key_cache.scalar_type() == query.scalar_type(), "the caches must be FP8-e4m3 or have the query's dtype");
  TORCH_CHECK(key_cache.dim() == 4 && value_cache.sizes() == key_cache.sizes() &&
                  value_cache.scalar_type() == key_cache.scalar_type() && key_cache.stride(3) == 1 &&
                  value_cache.stride(3) == 1,
              "cache must use NHD [blocks, block, heads, dim]");
  TORCH_CHECK(key_cache.size(2) == key.size(1) && key_cache.size(3) == key.size(2), "cache head shape must match K/V");
  TORCH_CHECK(positions.scalar_type() == at::kLong && slot_mapping.scalar_type() == at::kLong &&
                  positions.is_contiguous() && slot_mapping.is_contiguous() && positions.numel() == query.size(0) &&
                  slot_mapping.numel() == query.size(0),
              "positions and slot_mapping must match token count");
  TORCH_CHECK(cos_sin_cache.dim() == 2 && cos_sin_cache.stride(1) == 1 &&
                  (cos_sin_cache.scalar_type() == at::kFloat || cos_sin_cache.scalar_type() == query.scalar_type()),
              "cos_sin_cache must be [max_position, rotary_dim] in float32 or the query's dtype");
  pfd_rope_args a{};
  a.struct_size = sizeof(a);
  a.num_tokens = static_cast<int32_t>(query.size(0));
  a.num_q_heads = static_cast<int32_t>(query.size(1));
  a.num_kv_heads = static_cast<int32_t>(key.size(1));
  a.head_dim = static_cast<int32_t>(query.size(2));
  a.rotary_dim = static_cast<int32_t>(cos_sin_cache.size(1));
  a.block_size = static_cast<int32_t>(key_cache.size(1));
  a.is_neox = is_neox ? 1 : 0;
  a.query_dtype = dtype_code(query.scalar_type(), "query");
  a.cos_sin_dtype = cos_sin_cache.scalar_type() == at::kFloat ? PFD_DTYPE_F32 : a.query_dtype;
  a.cache_dtype = fp8 ? PFD_DTYPE_E4M3 : a.query_dtype;
  a.query = query.data_ptr(); a.q_stride_t = query.stride(0); a.q_stride_h = query.stride(1);
  a.key = key.data_ptr(); a.k_stride_t = key.stride(0); a.k_stride_h = key.stride(1);
  a.value = value.data_ptr(); a.v_stride_t = value.stride(0); a.v_stride_h = value.stride(1);
  a.positions = positions.data_ptr<int64_t>();
  a.cos_sin_cache = cos_sin_cache.data_ptr();
  a.cos_sin_stride = cos_sin_cache.stride(0);
  a.slot_mapping = slot_mapping.data_ptr<int64_t>();
  a.key_cache = key_cache.data_ptr();
  a.kc_stride_block = key_cache.stride(0); a.kc_stride_token = key_cache.stride(1); a.kc_stride_head = key_cache.stride(2);
  a.value_cache = value_cache.data_ptr();
  a.vc_stride_block = value_cache.stride(0); a.vc_stride_token = value_cache.stride(1); a.vc_stride_head = value_cache.stride(2);
  a.k_scale = a.v_scale = 1.0f;
  if (fp8) {
    TORCH_CHECK(k_scale.has_value() && v_scale.has_value(), "FP8 caches need k_scale and v_scale");
    for (const at::Tensor* s : {&*k_scale, &*v_scale})
      TORCH_CHECK(s->is_cuda() && s->scalar_type() == at::kFloat && s->is_contiguous() && s->numel() == key.size(1),
                  "scales must be float32 CUDA tensors with one entry per KV head");
    a.k_scale_per_head = k_scale->data_ptr<float>();
    a.v_scale_per_head = v_scale->data_ptr<float>();
  }
  const at::cuda::CUDAGuard guard(query.device());
  a.stream = at::cuda::getCurrentCUDAStream().stream();
  TORCH_CHECK(pfd_rope_quant_append(&a) == PFD_OK, pfd_last_error());
}

void merge_packed_partials(at::Tensor packed, at::Tensor output) {
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kFloat && packed.is_contiguous() &&
                  packed.dim() == 4,
              "packed must be contiguous float32 [parts, B, Hq, D + 2]");
  const int64_t d = packed.size(3) - 2;
  TORCH_CHECK(output.is_cuda() && output.is_contiguous() && output.dim() == 3 &&
                  output.size(0) == packed.size(1) && output.size(1) == packed.size(2) &&
                  output.size(2) == d,
              "output must be contiguous [B, Hq, D]");
  const at::cuda::CUDAGuard guard(packed.device());
  const int rc = pfd_merge_packed(packed.data_ptr<float>(), static_cast<int32_t>(packed.size(0)),
                                  packed.size(1) * packed.size(2), static_cast<int32_t>(d),
                                  output.data_ptr(), dtype_code(output.scalar_type(), "output"),
                                  at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == PFD_OK, pfd_last_error());
}

void resolve_slots(at::Tensor block_table, at::Tensor seq_lens, at::Tensor slots) {
  TORCH_CHECK(block_table.is_cuda() && block_table.scalar_type() == at::kInt && block_table.dim() == 2 &&
                  block_table.stride(1) == 1,
              "int32 block table");
  TORCH_CHECK(seq_lens.is_cuda() && seq_lens.scalar_type() == at::kInt && seq_lens.is_contiguous(),
              "int32 sequence lengths");
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kLong && slots.is_contiguous() &&
                  slots.dim() == 2 && slots.size(0) == block_table.size(0) &&
                  slots.size(1) <= block_table.size(1) * 16,
              "slots must be contiguous int64 [B, max_seq_len]");
  const at::cuda::CUDAGuard guard(block_table.device());
  const int rc = pfd_resolve_slots(block_table.data_ptr<int32_t>(), block_table.stride(0),
                                   seq_lens.data_ptr<int32_t>(), static_cast<int32_t>(slots.size(0)),
                                   static_cast<int32_t>(slots.size(1)), slots.data_ptr<int64_t>(),
                                   at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == PFD_OK, pfd_last_error());
}

int64_t prefix_groups_bytes(int64_t batch, int64_t max_groups) {
  const int64_t n = pfd_prefix_groups_bytes(static_cast<int32_t>(batch), static_cast<int32_t>(max_groups));
  TORCH_CHECK(n >= 0, pfd_last_error());
  return n;
}

void group_shared_prefixes(at::Tensor block_table, c10::optional<at::Tensor> prefix_lengths, int64_t uniform_prefix_len,
                           c10::optional<at::Tensor> seq_lens, int64_t min_batch, int64_t min_prefix_len,
                           int64_t max_groups, at::Tensor groups) {
  TORCH_CHECK(block_table.is_cuda() && block_table.scalar_type() == at::kInt && block_table.dim() == 2 &&
                  block_table.stride(1) == 1,
              "int32 block table");
  const int64_t batch = block_table.size(0);
  const int32_t* lengths = nullptr;
  const int32_t* lens = nullptr;
  if (prefix_lengths.has_value()) {
    TORCH_CHECK(prefix_lengths->is_cuda() && prefix_lengths->scalar_type() == at::kInt &&
                    prefix_lengths->is_contiguous() && prefix_lengths->numel() == batch,
                "prefix_lengths must be int32 CUDA with one entry per request");
    lengths = prefix_lengths->data_ptr<int32_t>();
  }
  if (seq_lens.has_value()) {
    TORCH_CHECK(seq_lens->is_cuda() && seq_lens->scalar_type() == at::kInt && seq_lens->is_contiguous() &&
                    seq_lens->numel() == batch,
                "int32 sequence lengths");
    lens = seq_lens->data_ptr<int32_t>();
  }
  TORCH_CHECK(groups.is_cuda() && groups.scalar_type() == at::kInt && groups.is_contiguous(),
              "groups must be a contiguous int32 CUDA tensor");
  const at::cuda::CUDAGuard guard(block_table.device());
  const int rc = pfd_group_shared_prefixes(
      block_table.data_ptr<int32_t>(), block_table.stride(0), static_cast<int32_t>(block_table.size(1)), lengths,
      static_cast<int32_t>(uniform_prefix_len), lens, static_cast<int32_t>(batch), static_cast<int32_t>(min_batch),
      static_cast<int32_t>(min_prefix_len), static_cast<int32_t>(max_groups), groups.data_ptr<int32_t>(),
      groups.numel() * 4, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == PFD_OK, pfd_last_error());
}

}  // namespace

TORCH_LIBRARY(l20_stack, module) {
  module.def(
      "paged_decode_split_out("
      "Tensor query, Tensor key_cache, Tensor value_cache, "
      "Tensor block_table, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, "
      "Tensor(c!) partial_sum, Tensor(d!) output, "
      "int max_seq_len, int split_size) -> Tensor(d!)");
  module.def(
      "paged_decode_split_out_v2("
      "Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, Tensor(c!) partial_sum, Tensor(d!) output, "
      "int max_seq_len, int split_size, int flags, Tensor(e!)? plan) -> ()");
  module.def(
      "paged_decode_split_indices_out("
      "Tensor query, Tensor key_cache, Tensor value_cache, "
      "Tensor page_indptr, Tensor page_indices, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, "
      "Tensor(c!) partial_sum, Tensor(d!) output, "
      "int max_seq_len, int split_size) -> ()");
  module.def(
      "paged_decode_fp8_e4m3_split_out("
      "Tensor query, Tensor key_cache, Tensor value_cache, "
      "Tensor block_table, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, "
      "Tensor(c!) partial_sum, Tensor(d!) output, "
      "float k_scale, float v_scale, "
      "int max_seq_len, int split_size) -> Tensor(d!)");
  module.def(
      "paged_decode_fp8_e4m3_split_out_v2("
      "Tensor query, Tensor key_cache, Tensor value_cache, "
      "Tensor block_table, Tensor seq_lens, "
      "Tensor(a!)? partial_output, Tensor(b!)? partial_max, "
      "Tensor(c!)? partial_sum, Tensor(d!)? output, Tensor(e!)? packed_output, "
      "Tensor k_scale, Tensor v_scale, float sm_scale, "
      "int max_seq_len, int split_size, int kv_start, int flags, Tensor(f!)? plan) -> ()");
  module.def(
      "plan_decode(Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor seq_lens, "
      "Tensor partial_output, Tensor partial_max, Tensor partial_sum, Tensor(a!) plan, "
      "int max_seq_len, int split_size, int kv_start) -> ()");
  module.def(
      "shared_prefix_decode_fp8_e4m3("
      "Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, Tensor(c!) partial_sum, Tensor(d!) output, "
      "Tensor k_scale, Tensor v_scale, float sm_scale, int max_seq_len, int split_size, int prefix_len) -> ()");
  module.def(
      "shared_prefix_decode_grouped_fp8_e4m3("
      "Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor seq_lens, "
      "Tensor(a!) partial_output, Tensor(b!) partial_max, Tensor(c!) partial_sum, Tensor(d!) output, "
      "Tensor k_scale, Tensor v_scale, float sm_scale, int max_seq_len, int split_size, Tensor groups, "
      "int max_groups, int max_prefix_len, int max_suffix_len, bool all_in_groups=False) -> ()");
  module.def(
      "rope_and_cache(Tensor(a!) query, Tensor(b!) key, Tensor value, Tensor positions, Tensor cos_sin_cache, "
      "bool is_neox, Tensor(c!) key_cache, Tensor(d!) value_cache, Tensor slot_mapping, "
      "Tensor? k_scale, Tensor? v_scale) -> ()");
  module.def("plan_bytes(int batch, int num_kv_heads) -> int", &plan_bytes);
  module.def("merge_packed_partials(Tensor packed, Tensor(a!) output) -> ()");
  module.def("resolve_slots(Tensor block_table, Tensor seq_lens, Tensor(a!) slots) -> ()");
  module.def("prefix_groups_bytes(int batch, int max_groups) -> int", &prefix_groups_bytes);
  module.def(
      "group_shared_prefixes(Tensor block_table, Tensor? prefix_lengths, int uniform_prefix_len, Tensor? seq_lens, "
      "int min_batch, int min_prefix_len, int max_groups, Tensor(a!) groups) -> ()");
}

TORCH_LIBRARY_IMPL(l20_stack, CUDA, module) {
  module.impl("paged_decode_split_out", &paged_decode_split_out);
  module.impl("paged_decode_split_out_v2", &paged_decode_split_out_v2);
  module.impl("paged_decode_split_indices_out", &paged_decode_split_indices_out);
  module.impl("paged_decode_fp8_e4m3_split_out", &paged_decode_fp8_e4m3_split_out);
  module.impl("paged_decode_fp8_e4m3_split_out_v2", &paged_decode_fp8_e4m3_split_out_v2);
  module.impl("plan_decode", &plan_decode);
  module.impl("shared_prefix_decode_fp8_e4m3", &shared_prefix_decode_fp8_e4m3);
  module.impl("rope_and_cache", &rope_and_cache);
  module.impl("merge_packed_partials", &merge_packed_partials);
  module.impl("resolve_slots", &resolve_slots);
  module.impl("shared_prefix_decode_grouped_fp8_e4m3", &shared_prefix_decode_grouped_fp8_e4m3);
  module.impl("group_shared_prefixes", &group_shared_prefixes);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) {
  module.def("paged_decode_split_out", &paged_decode_split_out_void);
  module.def("paged_decode_split_indices_out", &paged_decode_split_indices_out);
  module.def("paged_decode_fp8_e4m3_split_out", &paged_decode_fp8_e4m3_split_out_void);
  module.def("launch_count", []() { return pfd_launch_count(); });
}
