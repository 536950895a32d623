// C ABI of libpaged_fp8_decode.so: argument checks, kernel selection, launches.
// Declarations and reference citations: include/paged_fp8_decode.h.
#include "paged_fp8_decode.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>

#include "paged_decode_kernels.cuh"

namespace {

thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return PFD_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kWarps = 4;

template <int D, bool QBF16>
int launch_decode(const pfd_decode_args& a, const pfd::KernelParams& kp, int num_splits) {
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  const dim3 grid(num_splits, a.num_kv_heads, a.batch);
  pfd::paged_decode_fp8_partial_ldg_kernel<D, QBF16, kWarps><<<grid, kWarps * 32, 0, stream>>>(kp);
  if (int rc = check_launch("partial kernel")) return rc;
  if ((num_splits > 1 || !kp.direct_out) && !(a.flags & PFD_FLAG_PARTIAL_ONLY)) {
    const int rows = a.batch * a.num_q_heads;
    pfd::paged_decode_merge_kernel<D, QBF16><<<(rows + 3) / 4, 128, 0, stream>>>(kp, a.batch);
    if (int rc = check_launch("merge kernel")) return rc;
  }
  return PFD_OK;
}

}  // namespace

extern "C" {

int pfd_abi_version(void) { return PFD_ABI_VERSION; }

const char* pfd_last_error(void) { return g_last_error.c_str(); }

int64_t pfd_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int pfd_paged_decode_fp8_e4m3_split_out(const pfd_decode_args* args) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu",
                args->struct_size, sizeof(pfd_decode_args));
  const pfd_decode_args& a = *args;
  if (a.batch < 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0)
    return fail(PFD_ERR_INVALID, "invalid query");
  if (a.head_dim != 64 && a.head_dim != 128)
    return fail(PFD_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
  if (a.page_size != pfd::kPage) return fail(PFD_ERR_UNSUPPORTED, "page_size must be 16");
  if (a.num_q_heads % a.num_kv_heads != 0)
    return fail(PFD_ERR_INVALID, "Q heads must be divisible by KV heads");
  const int group = a.num_q_heads / a.num_kv_heads;
  if (group > 16) return fail(PFD_ERR_UNSUPPORTED, "at most 16 query heads per KV head");
  if (a.query_dtype != PFD_DTYPE_F16 && a.query_dtype != PFD_DTYPE_BF16)
    return fail(PFD_ERR_INVALID, "query must be FP16 or BF16");
  if (a.split_size < 16 || a.split_size % 16 != 0)
    return fail(PFD_ERR_INVALID, "split_size must be a multiple of 16");
  if (a.kv_start < 0 || a.max_seq_len < 0) return fail(PFD_ERR_INVALID, "negative length");
  if (a.batch == 0) return PFD_OK;
  if (!a.query || !a.key_cache || !a.value_cache || !a.block_table || !a.seq_lens)
    return fail(PFD_ERR_INVALID, "NULL operand");
  if (!a.output && !a.packed_output) return fail(PFD_ERR_INVALID, "no output given");
  if (a.q_stride_h % 4 || a.q_stride_b % 4 || (reinterpret_cast<uintptr_t>(a.query) & 7u))
    return fail(PFD_ERR_UNSUPPORTED, "query rows must be 8-byte aligned");
  if (a.output && (a.o_stride_h % 4 || a.o_stride_b % 4 || (reinterpret_cast<uintptr_t>(a.output) & 7u)))
    return fail(PFD_ERR_UNSUPPORTED, "output rows must be 8-byte aligned");
  if (!aligned16(a.key_cache) || !aligned16(a.value_cache) || a.k_stride_page % 16 ||
      a.k_stride_token % 16 || a.k_stride_head % 16 || a.v_stride_page % 16 ||
      a.v_stride_token % 16 || a.v_stride_head % 16)
    return fail(PFD_ERR_UNSUPPORTED, "K/V cache base and strides must be multiples of 16 bytes");

  const int span = a.max_seq_len > a.kv_start ? a.max_seq_len - a.kv_start : 0;
  int num_splits = (span + a.split_size - 1) / a.split_size;
  if (num_splits < 1) num_splits = 1;
  const bool direct_ok = !(a.flags & PFD_FLAG_NO_DIRECT_OUT);
  if (num_splits > 1 || !direct_ok) {
    if (!a.partial_output || !a.partial_max || !a.partial_sum)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape");
    if (a.workspace_splits < num_splits)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape");
    if (a.partial_dtype < PFD_DTYPE_F32 || a.partial_dtype > PFD_DTYPE_BF16)
      return fail(PFD_ERR_INVALID, "partial_output dtype must be f32, f16 or bf16");
    if (!aligned16(a.partial_output))
      return fail(PFD_ERR_UNSUPPORTED, "partial_output must be 16-byte aligned");
  }

  pfd::KernelParams kp{};
  kp.query = a.query;
  kp.key_cache = static_cast<const uint8_t*>(a.key_cache);
  kp.value_cache = static_cast<const uint8_t*>(a.value_cache);
  kp.block_table = a.block_table;
  kp.seq_lens = a.seq_lens;
  kp.k_scale_ph = a.k_scale_per_head;
  kp.v_scale_ph = a.v_scale_per_head;
  kp.partial_output = a.partial_output;
  kp.partial_max = a.partial_max;
  kp.partial_sum = a.partial_sum;
  kp.output = a.output;
  kp.packed_output = a.packed_output;
  kp.q_stride_b = a.q_stride_b; kp.q_stride_h = a.q_stride_h;
  kp.k_stride_page = a.k_stride_page; kp.k_stride_token = a.k_stride_token; kp.k_stride_head = a.k_stride_head;
  kp.v_stride_page = a.v_stride_page; kp.v_stride_token = a.v_stride_token; kp.v_stride_head = a.v_stride_head;
  kp.bt_stride_b = a.bt_stride_b;
  kp.partial_stride_b = a.partial_stride_b; kp.partial_stride_h = a.partial_stride_h;
  kp.partial_stride_s = a.partial_stride_s;
  kp.o_stride_b = a.o_stride_b; kp.o_stride_h = a.o_stride_h;
  kp.k_scale = a.k_scale; kp.v_scale = a.v_scale;
  kp.sm_scale = a.sm_scale != 0.f ? a.sm_scale : 1.0f / sqrtf(static_cast<float>(a.head_dim));
  kp.num_q_heads = a.num_q_heads; kp.num_kv_heads = a.num_kv_heads; kp.group = group;
  kp.split_size = a.split_size; kp.kv_start = a.kv_start;
  kp.partial_dtype = a.partial_dtype;
  kp.direct_out = direct_ok ? 1 : 0;

  const bool bf16 = a.query_dtype == PFD_DTYPE_BF16;
  if (a.head_dim == 128)
    return bf16 ? launch_decode<128, true>(a, kp, num_splits) : launch_decode<128, false>(a, kp, num_splits);
  return bf16 ? launch_decode<64, true>(a, kp, num_splits) : launch_decode<64, false>(a, kp, num_splits);
}

// ---- allocation-free entry point -------------------------------------------------------
// The partial workspace of the split-KV path as a fixed array in the library image.  In host
// code the name below is only a stand-in for the symbol, never a device address: the address
// each device uses comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PFD_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

int pfd_paged_decode_fp8_e4m3_split_out_noalloc(const pfd_decode_args* args) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu",
                args->struct_size, sizeof(pfd_decode_args));
  pfd_decode_args a = *args;
  if (a.batch < 0 || a.num_q_heads <= 0 || a.head_dim <= 0 || a.split_size < 16 || a.kv_start < 0 ||
      a.max_seq_len < 0)
    return fail(PFD_ERR_INVALID, "invalid geometry");
  const int64_t span = a.max_seq_len > a.kv_start ? a.max_seq_len - a.kv_start : 0;
  int64_t splits = (span + a.split_size - 1) / a.split_size;
  if (splits < 1) splits = 1;
  const int64_t rows = (int64_t)a.batch * a.num_q_heads * splits;
  const int64_t need = rows * (a.head_dim + 2) * (int64_t)sizeof(float);
  if (need > (int64_t)PFD_NOALLOC_SCRATCH_BYTES)
    return fail(PFD_ERR_UNSUPPORTED,
                "request needs %lld bytes of split-KV scratch but the built-in array holds %u; "
                "raise split_size or use the entry point that takes a workspace",
                (long long)need, PFD_NOALLOC_SCRATCH_BYTES);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(PFD_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(PFD_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev,
                    cudaGetErrorString(e));
      g_noalloc_ptr[dev] = p;
    }
    base = g_noalloc_ptr[dev];
  }
  float* po = static_cast<float*>(base);
  a.partial_output = po;
  a.partial_max = po + rows * a.head_dim;
  a.partial_sum = po + rows * a.head_dim + rows;
  a.partial_dtype = PFD_DTYPE_F32;
  a.workspace_splits = static_cast<int32_t>(splits);
  a.partial_stride_b = (int64_t)a.num_q_heads * splits;
  a.partial_stride_h = splits;
  a.partial_stride_s = 1;
  return pfd_paged_decode_fp8_e4m3_split_out(&a);
}

int pfd_merge_packed(const float* packed, int32_t num_parts, int64_t rows, int32_t head_dim,
                     void* output, int32_t out_dtype, void* stream) {
  if (!packed || !output) return fail(PFD_ERR_INVALID, "NULL operand");
  if (num_parts < 1 || rows < 0) return fail(PFD_ERR_INVALID, "invalid part or row count");
  if (head_dim != 64 && head_dim != 128) return fail(PFD_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
  if (out_dtype < PFD_DTYPE_F32 || out_dtype > PFD_DTYPE_BF16)
    return fail(PFD_ERR_INVALID, "output dtype must be f32, f16 or bf16");
  if (rows == 0) return PFD_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
  if (head_dim == 128)
    pfd::merge_packed_kernel<128><<<blocks, 128, 0, s>>>(packed, num_parts, rows, output, out_dtype);
  else
    pfd::merge_packed_kernel<64><<<blocks, 128, 0, s>>>(packed, num_parts, rows, output, out_dtype);
  return check_launch("merge_packed kernel");
}

int pfd_resolve_slots(const int32_t* block_table, int64_t bt_stride_b, const int32_t* seq_lens,
                      int32_t batch, int32_t max_seq_len, int64_t* slots, void* stream) {
  if (!block_table || !seq_lens || !slots) return fail(PFD_ERR_INVALID, "NULL operand");
  if (batch < 0 || max_seq_len < 0) return fail(PFD_ERR_INVALID, "negative size");
  if (batch == 0 || max_seq_len == 0) return PFD_OK;
  const dim3 grid((max_seq_len + 255) / 256, batch);
  pfd::resolve_slots_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      block_table, bt_stride_b, seq_lens, max_seq_len, slots);
  return check_launch("resolve_slots kernel");
}

}  // extern "C"
