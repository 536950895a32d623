// C ABI of libpaged_fp8_decode.so: argument checks, kernel selection, launches.
// Declarations and reference citations: include/paged_fp8_decode.h.
#include "paged_fp8_decode.h"

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "paged_decode_balanced.cuh"
#include "shared_prefix_dense.cuh"
#include "paged_decode_kernels.cuh"
#include "rope_kv_append.cuh"
#include "shared_prefix_groups.cuh"

namespace {

thread_local std::string g_last_error;
thread_local int g_last_path = 0;  // PFD_PATH_* of this thread's last decode call
unsigned long long* g_phase_times = nullptr;  // tuning builds (-DPFD_PHASE_STAMPS) only: stamp buffer
std::atomic<int64_t> g_launches{0};
// How long a device-side wait for a copy may last before it gives up (pfd_set_wait_limit_ns).
std::atomic<unsigned long long> g_wait_limit_ns{200ull * 1000 * 1000};

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
constexpr int kStages = 2;
constexpr int kMaxDevices = 64;

// Error word the kernels write (bounded waits that gave up).  The name is a host-side stand-in
// for the symbol; each device's address is looked up once with cudaGetSymbolAddress.
static __device__ int g_device_status;
std::mutex g_state_mutex;

// What a call needs to know about its device, looked up once per device.  Every entry point
// begins with enter_call(): one cudaGetDevice, then a lock-free read of this table; the helpers
// below take the device of the call in progress from t_device.
struct DeviceState {
  int dev = -1;
  int sms = 0;
  int32_t* status = nullptr;
};
DeviceState g_device_state[kMaxDevices];
std::atomic<bool> g_device_ready[kMaxDevices];
thread_local const DeviceState* t_device = nullptr;

int enter_call() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(PFD_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (!g_device_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_state_mutex);
    if (!g_device_ready[dev].load(std::memory_order_relaxed)) {
      DeviceState& d = g_device_state[dev];
      e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_device_status);
      if (e != cudaSuccess || p == nullptr)
        return fail(PFD_ERR_CUDA, "cudaGetSymbolAddress(status) failed: %s", cudaGetErrorString(e));
      d.status = static_cast<int32_t*>(p);
      d.dev = dev;
      g_device_ready[dev].store(true, std::memory_order_release);
    }
  }
  t_device = &g_device_state[dev];
  return PFD_OK;
}

int status_pointer(int32_t** out) {
  *out = t_device->status;
  return PFD_OK;
}

// First launch of a kernel that needs more than the default dynamic shared memory, per device.
// `whole_sm`: also ask for the largest shared-memory carve-out, so that a CTA of another kernel
// can use what this one leaves over (the carve-out is otherwise sized for this kernel alone).
template <typename Kernel>
int configure_smem(std::atomic<bool>* done, Kernel kernel, int smem, bool whole_sm = false) {
  std::atomic<bool>& flag = done[t_device->dev];
  if (flag.load(std::memory_order_acquire)) return PFD_OK;
  std::lock_guard<std::mutex> lock(g_state_mutex);
  if (!flag.load(std::memory_order_relaxed)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess && whole_sm)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    flag.store(true, std::memory_order_release);
  }
  return PFD_OK;
}

// ---- tensor maps (TMA descriptors) of the K and V caches, cached per distinct cache view ----
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

struct MapKey {
  int dev;
  const void* base;
  int64_t stride_page, stride_token, stride_head, num_pages;
  int32_t heads;
  int32_t promotion;   // L2 promotion in bytes
  int32_t elem_bytes;  // 1: e4m3, 2: fp16 / bf16
  bool operator==(const MapKey& o) const {
    return dev == o.dev && base == o.base && stride_page == o.stride_page && stride_token == o.stride_token &&
           stride_head == o.stride_head && num_pages == o.num_pages && heads == o.heads &&
           promotion == o.promotion && elem_bytes == o.elem_bytes;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};
std::vector<MapEntry> g_maps;  // every map encoded so far (under g_state_mutex)
EncodeTiledFn g_encode = nullptr;
// Hit path: a direct-mapped table per thread, indexed by a hash of the cache's base address; no
// lock, one key comparison, one 128-byte copy.  A model's layers each have their own K and V
// cache, so a serving thread cycles through a few dozen entries.
constexpr int kMapSlots = 256;
struct MapSlot {
  bool used = false;
  MapEntry entry;
};
thread_local MapSlot t_map_slots[kMapSlots];
inline unsigned map_slot_of(const void* base, int32_t elem_bytes) {
  uint64_t x = reinterpret_cast<uintptr_t>(base) >> 8;
  x ^= x >> 17;
  x *= 0x9E3779B97F4A7C15ull;
  return (unsigned)((x >> 40) + (unsigned)elem_bytes) % kMapSlots;
}

bool head_is_dim1(int64_t stride_token, int64_t stride_head) { return stride_head <= stride_token; }

// [pages, 16, heads, 128] e4m3 bytes with arbitrary (page, token, head) strides as a rank-4 u8
// tensor whose dimensions are listed by ascending stride; box = one (page, head) tile of
// 16 x 128 bytes, 128-byte swizzle.
//
// L2 promotion: the fixed-split grid runs the CTAs of all kv heads of a page at about the same
// time, so fetching 256 bytes (two heads' rows in the NHD layout) per 128-byte request pays; the
// balanced grid does not keep kv heads in step, there the second half would be evicted unused.
// (With 2-byte elements the strides are given in elements and the box is half a row, 64
// elements = 128 bytes, so that the 128-byte swizzle still applies.)
int get_tensor_map(const void* base, int64_t stride_page, int64_t stride_token, int64_t stride_head,
                   int64_t num_pages, int32_t heads, int32_t promotion, CUtensorMap* out, int32_t elem_bytes = 1) {
  const MapKey key{t_device->dev, base, stride_page, stride_token, stride_head, num_pages, heads, promotion, elem_bytes};
  MapSlot& slot = t_map_slots[map_slot_of(base, elem_bytes)];
  if (slot.used && slot.entry.key == key) {
    *out = slot.entry.map;
    return PFD_OK;
  }
  std::lock_guard<std::mutex> lock(g_state_mutex);
  for (const MapEntry& e : g_maps)
    if (e.key == key) {
      slot.entry = e;
      slot.used = true;
      *out = e.map;
      return PFD_OK;
    }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr)
      return fail(PFD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const bool h1 = head_is_dim1(stride_token, stride_head);
  const cuuint64_t dims[4] = {128, (cuuint64_t)(h1 ? heads : 16), (cuuint64_t)(h1 ? 16 : heads),
                              (cuuint64_t)num_pages};
  const cuuint64_t strides[3] = {(cuuint64_t)(h1 ? stride_head : stride_token) * elem_bytes,
                                 (cuuint64_t)(h1 ? stride_token : stride_head) * elem_bytes,
                                 (cuuint64_t)stride_page * elem_bytes};
  const cuuint32_t box[4] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)(h1 ? 1 : 16), (cuuint32_t)(h1 ? 16 : 1), 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  MapEntry entry;
  entry.key = key;
  const CUtensorMapL2promotion promo =
      promotion == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                     : promotion == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                       : promotion == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                          : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  const CUresult r = g_encode(&entry.map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                              4, const_cast<void*>(base), dims, strides,
                              box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PFD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  if (g_maps.size() >= 1024) g_maps.erase(g_maps.begin());
  g_maps.push_back(entry);
  slot.entry = entry;
  slot.used = true;
  *out = entry.map;
  return PFD_OK;
}

bool tma_eligible(const pfd_decode_args& a) {
  if (a.head_dim != 128 || (a.flags & PFD_FLAG_NO_TMA)) return false;
  // a size-1 dimension may carry any stride; everything else was checked to be 16-byte aligned
  return a.k_stride_page > 0 && a.v_stride_page > 0 && a.k_stride_token > 0 && a.v_stride_token > 0 &&
         a.k_stride_head > 0 && a.v_stride_head > 0 && a.num_pages > 0 &&
         head_is_dim1(a.k_stride_token, a.k_stride_head) == head_is_dim1(a.v_stride_token, a.v_stride_head);
}

// kWarpsT = 2, kStagesT = 1 beside the dense prefix pass: two CTAs of two warps, 165 registers
// and 18 KB fit on an SM next to a CTA of the slim prefix kernel (see suffix_beside_prefix).
template <bool QBF16, int kWarpsT = kWarps, int kStagesT = kStages>
int launch_partial_tma(const pfd_decode_args& a, const pfd::KernelParams& kp, dim3 grid, cudaStream_t stream) {
  CUtensorMap mk, mv;
  if (int rc = get_tensor_map(a.key_cache, a.k_stride_page, a.k_stride_token, a.k_stride_head, a.num_pages,
                              a.num_kv_heads, 256, &mk))
    return rc;
  if (int rc = get_tensor_map(a.value_cache, a.v_stride_page, a.v_stride_token, a.v_stride_head, a.num_pages,
                              a.num_kv_heads, 256, &mv))
    return rc;
  pfd::TmaParams tp{};
  tp.head_is_dim1 = head_is_dim1(a.k_stride_token, a.k_stride_head) ? 1 : 0;
  if (int rc = status_pointer(&tp.status)) return rc;
  tp.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  auto kernel = pfd::paged_decode_fp8_partial_tma_kernel<QBF16, kWarpsT, kStagesT>;
  constexpr int smem = 1024 + kWarpsT * kStagesT * 8192 + kWarpsT * kStagesT * 8 + 2 * kWarpsT * 16 * 4;
  static std::atomic<bool> configured[kMaxDevices];  // (one array per instantiation)
  if (int rc = configure_smem(configured, kernel, smem, kWarpsT != kWarps)) return rc;
  {
    // Programmatic dependent launch.  Behind the dense prefix pass: independent work, it runs
    // beside that pass.  Otherwise: the CTAs may become resident while the preceding kernel of
    // the stream drains; the kernel waits for that kernel's completion before its first access.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarpsT * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, kp, tp, mk, mv);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "partial kernel (TMA) launch failed: %s", cudaGetErrorString(e));
  }
  return check_launch("partial kernel (TMA)");
}

// Behind the dense prefix pass the split-KV pass has two forms.  Two-warp CTAs with a one-stage
// ring (165 registers, 18 KB) fit BESIDE a CTA of the slim dense kernel -- two per SM there, six
// on an SM that pass leaves free -- and run while it runs.  Otherwise the ordinary four-warp CTAs
// are launched behind the dense pass; as its programmatic dependents they start, three per SM, on
// whatever SMs the last wave of that pass leaves free, and only what those SMs do not get done
// while the wave runs is left for afterwards.  The small form costs the dense pass 1 us and its
// CTAs are slow (two warps, one copy in flight each), so it is taken only when the free SMs
// cannot absorb the suffix work.  Measured in us per step (behind / beside), 16 query and 2 KV
// heads, prefix 4096 unless noted, suffixes up to 511 behind it (batch b = 2 b dense CTAs):
//   batch 64, splits of 128: 19.8 / 17.4   of 256: 21.7 / 19.2   of 512: 24.6 / 24.8
//   batch 16: 14.2 / 15.1   batch 32: 15.1 / 16.0   batch 48: 15.2 / 16.9   batch 96: 29.1 / 31.5
//   batch 128, splits of 128: 34.3 / 35.6   of 256: 35.5 / 34.2      batch 256, of 256: 59.8 / 65.3   of 512: 61.7 / 65.5
//   batch 64 with 3072 of the 4096 declared shared (96 CTAs, suffixes up to 1535, splits of 384): 23.8 / 21.9
//   ... 2048 declared (64 CTAs, suffixes up to 2559), splits of 512: 26.0 / 27.5   of 256: 28.4 / 27.6
//   batch 128 with 2048 declared (128 CTAs), splits of 512: 46.0 / 44.9
// The estimate below (a dense wave lasts 10 us, a four-warp CTA 2 us + 1 us per page pair of each
// warp, about 65 % of the grid has work; never with more than two dense waves, each of which
// pays the slim kernel's 1 us) decides all of these but one as measured.  A request in
// no group attends its whole context in as many splits as the others their suffix, which two
// warps would take several times longer over: with a groups table the small form needs the
// caller's word that every request is in a group (PFD_FLAG_ALL_IN_GROUPS).
std::atomic<int> g_suffix_form{-1};  // tuning: -1 choose, 0 always behind, 1 always beside
bool suffix_beside_prefix(const pfd_decode_args& a, int prefix_chunks, int num_splits, bool groups_table) {
  if (prefix_chunks <= 0 || a.head_dim != 128 || !tma_eligible(a)) return false;
  const int forced = g_suffix_form.load(std::memory_order_relaxed);
  if (forced >= 0) return forced == 1;
  if (groups_table && !(a.flags & PFD_FLAG_ALL_IN_GROUPS)) return false;
  const int group = a.num_q_heads / a.num_kv_heads;
  const int64_t dense_ctas = (int64_t)prefix_chunks * a.num_kv_heads *
                             (((int64_t)a.batch * group + pfd::kPrefixRows - 1) / pfd::kPrefixRows);
  const int64_t grid_ctas = (int64_t)num_splits * a.num_kv_heads * a.batch;
  if (grid_ctas * a.split_size > 6144 * dense_ctas) return false;  // suffixes far longer than the prefix
  const int sms = t_device->sms;
  if (dense_ctas > 2 * sms) return false;
  const int last_wave = dense_ctas % sms == 0 ? sms : static_cast<int>(dense_ctas % sms);
  const double cta_us = 2.0 + (a.split_size + 127) / 128;
  const double absorbed = 3.0 * (sms - last_wave) * (10.0 / cta_us);
  return 0.65 * static_cast<double>(grid_ctas) > absorbed;
}

// ---- balanced persistent kernel -------------------------------------------------------------
// Eight warps with three 8 KiB stages each keep 192 KiB per SM in flight; measured on B200 this
// beats twelve warps x two stages (smaller chunks, more pieces to merge) and six x four (the
// warps no longer keep up with the copies).
constexpr int kChunkStages = 3;
constexpr int kChunkWarps = 8;  // per CTA, one CTA per SM
constexpr int kChunkMaxBatch = 2048;
// 16-bit caches: a stage of two pages is 16 KiB, six warps x two stages fill the same 192 KiB.
constexpr int kChunkStages16 = 2;
constexpr int kChunkWarps16 = 6;
// Half page pairs charged for starting a sequence.  Measured on the batch-256 configuration
// (us per step): 0 -> 53.9, 1 -> 44.2, 2 -> 43.0, 3 -> 43.3, 4 -> 44.0; the batch-64 one does not care.
constexpr int kChunkPieceCost = 2;

bool balanced_eligible(const pfd_decode_args& a, int group, int slot_offset, int sms) {
  if (a.flags & (PFD_FLAG_FIXED_SPLITS | PFD_FLAG_NO_TMA | PFD_FLAG_NO_DIRECT_OUT)) return false;
  if (slot_offset != 0) return false;  // slots in front belong to the dense prefix pass
  if (a.head_dim != 128 || !tma_eligible(a) || group > 8 || a.batch > kChunkMaxBatch) return false;
  if (a.num_kv_heads > kChunkWarps * sms / 2) return false;  // one warp per kv head and group
  if (!a.partial_output || !a.partial_max || !a.partial_sum || a.partial_dtype != PFD_DTYPE_F32) return false;
  if (a.partial_stride_s != 1 || a.partial_stride_h != a.workspace_splits ||
      a.partial_stride_b != (int64_t)a.num_q_heads * a.workspace_splits)
    return false;
  const int64_t rows = (int64_t)a.batch * a.num_q_heads * a.workspace_splits;
  return rows >= 2LL * (sms * kChunkWarps / a.num_kv_heads) * a.num_q_heads;
}

// Warps of the balanced grid that take part: all of them, or fewer when the workspace has room
// for fewer slots (max_groups > 0).  The plan is made for the same number.
int balanced_num_warps(int sms, int warps_per_cta, int num_kv_heads, int max_groups) {
  int n = sms * warps_per_cta;
  if (max_groups > 0) n = std::min(n, max_groups * num_kv_heads);
  return n;
}

// max_groups > 0 caps the number of warp groups (a workspace with room for fewer slots).
template <bool QBF16, int kStagesT, int kWarpsT, bool KV16 = false>
int launch_balanced(const pfd_decode_args& a, const pfd::KernelParams& kp, int sms, cudaStream_t stream,
                    int max_groups = 0) {
  CUtensorMap mk, mv;
  constexpr int kElem = KV16 ? 2 : 1;
  if (int rc = get_tensor_map(a.key_cache, a.k_stride_page, a.k_stride_token, a.k_stride_head, a.num_pages,
                              a.num_kv_heads, 256, &mk, kElem))
    return rc;
  if (int rc = get_tensor_map(a.value_cache, a.v_stride_page, a.v_stride_token, a.v_stride_head, a.num_pages,
                              a.num_kv_heads, 256, &mv, kElem))
    return rc;
  pfd::TmaParams tp{};
  tp.head_is_dim1 = head_is_dim1(a.k_stride_token, a.k_stride_head) ? 1 : 0;
  if (int rc = status_pointer(&tp.status)) return rc;
  tp.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  tp.phase_times = g_phase_times;
  // A plan needs f32 pieces (its in-kernel merge reads them as such; the merge kernel takes either).
  const bool planned = a.plan != nullptr && a.partial_dtype == PFD_DTYPE_F32;
  const bool fused = planned && (a.flags & PFD_FLAG_SINGLE_LAUNCH) && !(a.flags & PFD_FLAG_PARTIAL_ONLY);
  auto kernel = fused ? pfd::paged_decode_fp8_chunk_kernel<QBF16, kStagesT, kWarpsT, KV16, true>
                      : pfd::paged_decode_fp8_chunk_kernel<QBF16, kStagesT, kWarpsT, KV16, false>;
  constexpr int kThreads = kWarpsT * 32;
  // ring + mbarriers + scan scratch + prefix[B + 1] + lens[B], sized for the largest batch
  constexpr int smem = 1024 + kWarpsT * kStagesT * 8192 * kElem + kWarpsT * kStagesT * 8 +
                       kWarpsT * 4 + (2 * kChunkMaxBatch + 1) * 4 + 16;
  static std::atomic<bool> configured[2][kMaxDevices];  // one array per instantiation of this template
  if (int rc = configure_smem(configured[fused ? 1 : 0], kernel, smem)) return rc;
  pfd::ChunkParams cp{};
  cp.batch = a.batch;
  cp.num_warps = balanced_num_warps(sms, kWarpsT, a.num_kv_heads, max_groups);
  cp.piece_cost = kChunkPieceCost;
  cp.plan = planned ? static_cast<int32_t*>(a.plan) : nullptr;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, kp, tp, cp, mk, mv);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "balanced decode kernel launch failed: %s", cudaGetErrorString(e));
    if (int rc = check_launch("balanced decode kernel")) return rc;
  }
  g_last_path = fused ? (KV16 ? PFD_PATH_FUSED_KV16 : PFD_PATH_FUSED)
                      : (KV16 ? PFD_PATH_BALANCED_KV16 : PFD_PATH_BALANCED);
  if (fused || (a.flags & PFD_FLAG_PARTIAL_ONLY)) return PFD_OK;
  {
    // Few rows mean few, long sequences whose pieces are many: four warps then share a row,
    // which also puts more loads in flight per SM (64 registers, 8 CTAs per SM).  Many rows: one
    // warp per row, up to 16 pieces requested in one round trip (128 registers, 4 CTAs per SM):
    // most rows of a large batch have nothing to merge and leave at once, and the few long
    // sequences that were cut into a dozen pieces set the tail -- 44.9 -> 43.0 us per step on the
    // batch-256 configuration against 8 pieces per round at 8 CTAs per SM.
    // (CTAs of a single warp and row, all resident beside the chunk kernel, were measured
    // slower: 21.8 against 19.9 us per step on the batch-64 configuration.)
    const int rows = a.batch * a.num_q_heads;
    const bool wide = rows <= 8 * sms;  // (one warp per row on the batch-64 configuration: 21.0 against 19.9 us)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(wide ? rows : (rows + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e =
        wide ? cudaLaunchKernelEx(&cfg, pfd::paged_decode_chunk_merge_kernel<QBF16, 4, 4, 8>, kp, tp, cp)
             : cudaLaunchKernelEx(&cfg, pfd::paged_decode_chunk_merge_kernel<QBF16, 1, 16, 4>, kp, tp, cp);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "balanced merge kernel launch failed: %s", cudaGetErrorString(e));
  }
  return check_launch("balanced merge kernel");
}

template <int D, bool QBF16>
int launch_decode(const pfd_decode_args& a, const pfd::KernelParams& kp, int num_splits) {
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  if (D == 128) {
    const int sms = t_device->sms;
    if (balanced_eligible(a, kp.group, kp.slot_offset, sms)) return launch_balanced<QBF16, kChunkStages, kChunkWarps>(a, kp, sms, stream);
  }
  if (a.page_indptr != nullptr)
    return fail(PFD_ERR_UNSUPPORTED,
                "page_indptr addressing needs the balanced kernel (head_dim 128, at most 8 query heads per KV "
                "head, dense f32 workspace of pfd_balanced_workspace_rows() rows)");
  const dim3 grid(num_splits, a.num_kv_heads, a.batch);
  if (D == 128 && tma_eligible(a)) {
    g_last_path = PFD_PATH_FIXED_TMA;
    if (int rc = suffix_beside_prefix(a, kp.slot_offset, num_splits, kp.row_kv_start != nullptr)
                     ? launch_partial_tma<QBF16, 2, 1>(a, kp, grid, stream)
                     : launch_partial_tma<QBF16>(a, kp, grid, stream))
      return rc;
  } else {
    g_last_path = PFD_PATH_FIXED_LDG;
    pfd::paged_decode_fp8_partial_ldg_kernel<D, QBF16, kWarps><<<grid, kWarps * 32, 0, stream>>>(kp);
    if (int rc = check_launch("partial kernel")) return rc;
  }
  if ((num_splits > 1 || !kp.direct_out) && !(a.flags & PFD_FLAG_PARTIAL_ONLY)) {
    const int rows = a.batch * a.num_q_heads;
    // programmatic dependent launch: the merge grid is scheduled while the partial grid drains
    cudaLaunchConfig_t cfg{};
    // few rows and more than eight slots per row: four warps share a row (one round trip instead of several)
    const int sms = t_device->sms;
    const bool wide = rows <= 8 * sms && num_splits + kp.slot_offset > 8;
    cfg.gridDim = dim3(wide ? rows : (rows + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int batch = a.batch;
    const cudaError_t e = wide ? cudaLaunchKernelEx(&cfg, pfd::paged_decode_merge_kernel<D, QBF16, 4>, kp, batch)
                               : cudaLaunchKernelEx(&cfg, pfd::paged_decode_merge_kernel<D, QBF16, 1>, kp, batch);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "merge kernel launch failed: %s", cudaGetErrorString(e));
    if (int rc = check_launch("merge kernel")) return rc;
  }
  return PFD_OK;
}

}  // namespace

extern "C" {

int pfd_abi_version(void) { return PFD_ABI_VERSION; }

const char* pfd_last_error(void) { return g_last_error.c_str(); }

int64_t pfd_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"

namespace {
// What the grouped shared-prefix entry adds to a split-KV pass: per-request attend starts read on
// the device, their cap, the split size of requests in no group, and the grid's split count.
struct GroupedRows {
  const int32_t* row_kv_start = nullptr;
  int row_kv_cap = 0;
  int split_size_loner = 0;
  int num_splits = 0;
};

pfd::KernelParams fill_params(const pfd_decode_args& a, int group, bool direct_ok, int slot_offset,
                              const GroupedRows* grouped = nullptr) {
  pfd::KernelParams kp{};
  kp.query = a.query;
  kp.key_cache = static_cast<const uint8_t*>(a.key_cache);
  kp.value_cache = static_cast<const uint8_t*>(a.value_cache);
  kp.block_table = a.block_table;
  kp.seq_lens = a.seq_lens;
  kp.page_indptr = a.page_indptr;
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
  kp.bt_cols = (a.max_seq_len + pfd::kPage - 1) / pfd::kPage;  // rows are at least this wide
  kp.slot_offset = slot_offset;
  if (grouped != nullptr) {
    kp.row_kv_start = grouped->row_kv_start;
    kp.row_kv_cap = grouped->row_kv_cap;
    kp.split_size_loner = grouped->split_size_loner;
  }
  kp.early_metadata = (a.flags & PFD_FLAG_EARLY_METADATA) ? 1 : 0;
  kp.early_kv = (kp.early_metadata && (a.flags & PFD_FLAG_EARLY_KV)) ? 1 : 0;
  kp.kv_evict_first = 1;
  if (a.exchange != nullptr) {
    const pfd_exchange& x = *a.exchange;
    kp.xch_world = x.world;
    kp.xch_rank = x.rank;
    kp.xch_rows = a.batch * a.num_q_heads;
    for (int r = 0; r < x.world && r < 8; ++r) kp.xch_recv[r] = static_cast<unsigned long long*>(x.recv[r]);
    kp.xch_control = static_cast<uint32_t*>(x.control);
    kp.packed_output = static_cast<float*>(x.recv[x.rank]);  // non-NULL selects the packed form; the kernels address through xch_recv
    kp.output = nullptr;
  }
#ifdef PFD_BOUNDS_CHECK
  kp.dbg_ws_rows = (int64_t)a.batch * a.num_q_heads * a.workspace_splits;
  kp.dbg_batch = a.batch;
#endif
  return kp;
}

// slot_offset > 0: workspace slots [0, slot_offset) are filled by the dense prefix pass; the
// split-KV kernels then write behind them and the merge kernel covers both.
int decode_impl(const pfd_decode_args* args, int slot_offset, const GroupedRows* grouped = nullptr) {
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
  if (!a.output && !a.packed_output && !a.exchange) return fail(PFD_ERR_INVALID, "no output given");
  if (a.exchange != nullptr) {
    const pfd_exchange& x = *a.exchange;
    if (x.world < 1 || x.world > 8 || x.rank < 0 || x.rank >= x.world || !x.control)
      return fail(PFD_ERR_INVALID, "exchange: world 1..8, 0 <= rank < world and the control words are needed");
    for (int r = 0; r < x.world; ++r)
      if (!x.recv[r]) return fail(PFD_ERR_INVALID, "exchange: recv pointer of rank %d is NULL", r);
    if (slot_offset != 0 || (a.flags & (PFD_FLAG_SINGLE_LAUNCH | PFD_FLAG_PARTIAL_ONLY)))
      return fail(PFD_ERR_UNSUPPORTED, "exchange: not with the shared-prefix pass, PFD_FLAG_SINGLE_LAUNCH or PFD_FLAG_PARTIAL_ONLY");
    if (int rc = enter_call()) return rc;
    const int sms = t_device->sms;
    if (!balanced_eligible(a, group, 0, sms))
      return fail(PFD_ERR_UNSUPPORTED,
                  "exchange: needs the balanced kernel (head_dim 128, at most 8 query heads per KV head, TMA-describable "
                  "cache, dense f32 workspace of pfd_balanced_workspace_rows() rows, no fixed-split flags)");
  }
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
  if (grouped != nullptr) num_splits = grouped->num_splits;
  if (num_splits < 1) num_splits = 1;
  const bool direct_ok = !(a.flags & PFD_FLAG_NO_DIRECT_OUT) && slot_offset == 0;
  if (num_splits > 1 || !direct_ok) {
    if (!a.partial_output || !a.partial_max || !a.partial_sum)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape");
    if (a.workspace_splits < num_splits + slot_offset)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape");
    if (a.partial_dtype < PFD_DTYPE_F32 || a.partial_dtype > PFD_DTYPE_BF16)
      return fail(PFD_ERR_INVALID, "partial_output dtype must be f32, f16 or bf16");
    if (!aligned16(a.partial_output))
      return fail(PFD_ERR_UNSUPPORTED, "partial_output must be 16-byte aligned");
  }

  if (int rc = enter_call()) return rc;  // (argument errors above are reported without a device)
  const pfd::KernelParams kp = fill_params(a, group, direct_ok, slot_offset, grouped);

  const bool bf16 = a.query_dtype == PFD_DTYPE_BF16;
  if (a.head_dim == 128)
    return bf16 ? launch_decode<128, true>(a, kp, num_splits) : launch_decode<128, false>(a, kp, num_splits);
  return bf16 ? launch_decode<64, true>(a, kp, num_splits) : launch_decode<64, false>(a, kp, num_splits);
}

template <bool QBF16>
int launch_prefix(const pfd_decode_args& a, int prefix_len, int chunks, bool suffix_beside,
                  const int32_t* groups = nullptr, int max_groups = 0) {
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
  kp.q_stride_b = a.q_stride_b; kp.q_stride_h = a.q_stride_h;
  kp.k_stride_page = a.k_stride_page; kp.k_stride_token = a.k_stride_token; kp.k_stride_head = a.k_stride_head;
  kp.v_stride_page = a.v_stride_page; kp.v_stride_token = a.v_stride_token; kp.v_stride_head = a.v_stride_head;
  kp.bt_stride_b = a.bt_stride_b;
  kp.partial_stride_b = a.partial_stride_b; kp.partial_stride_h = a.partial_stride_h;
  kp.partial_stride_s = a.partial_stride_s;
  kp.k_scale = a.k_scale; kp.v_scale = a.v_scale;
  kp.sm_scale = a.sm_scale != 0.f ? a.sm_scale : 1.0f / sqrtf(128.f);
  kp.num_q_heads = a.num_q_heads; kp.num_kv_heads = a.num_kv_heads;
  kp.group = a.num_q_heads / a.num_kv_heads;
  pfd::PrefixParams pp{};
  pp.prefix_len = prefix_len;
  pp.batch = a.batch;
  pp.groups = groups;
  pp.groups_batch = a.batch;
  pp.max_groups = max_groups;
  if (int rc = status_pointer(&pp.status)) return rc;
  pp.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  pp.phase_times = g_phase_times;
  // the slim instantiation (80 registers, whole-SM carve-out) leaves room for the suffix pass's
  // two-warp CTAs on the same SM; it is 1 us slower by itself, so the other one runs otherwise
  auto kernel = suffix_beside ? pfd::shared_prefix_dense_kernel<QBF16, true> : pfd::shared_prefix_dense_kernel<QBF16, false>;
  constexpr int smem = 1024 + 160 * 1024 + 32 + 2 * 4 * 128 * 4;
  static std::atomic<bool> configured[2][kMaxDevices];
  if (int rc = configure_smem(configured[suffix_beside ? 1 : 0], kernel, smem, suffix_beside)) return rc;
  const int rows = a.batch * kp.group;
  const int tiles = (rows + pfd::kPrefixRows - 1) / pfd::kPrefixRows;
  // Grouped: every group's last 128-row tile may be ragged, so there can be up to one more tile
  // per group than the rows fill.  The kernel's CTAs take tile slots in turns, so any grid is
  // right; slots beyond `tiles` are added only while the grid stays within one CTA per SM, where
  // a CTA that finds its slot empty costs nothing.  (Beyond that every idle CTA waits for a whole
  // SM's shared memory, and the suffix pass, a programmatic dependent, starts only after the
  // last of them: 6 us late with 128 idle CTAs on the batch of 64.)
  const int spare = std::max(0, std::min(max_groups, t_device->sms / std::max(chunks * a.num_kv_heads, 1) - tiles));
  const dim3 grid = groups == nullptr ? dim3(chunks, tiles, a.num_kv_heads)
                                      : dim3(chunks * a.num_kv_heads, tiles + spare, 1);
  kernel<<<grid, 512, smem, static_cast<cudaStream_t>(a.stream)>>>(kp, pp);
  return check_launch("shared-prefix dense kernel");
}
}  // namespace

extern "C" {

int pfd_paged_decode_fp8_e4m3_split_out(const pfd_decode_args* args) { return decode_impl(args, 0); }

// ---- non-quantised sibling: caches in the query's 16-bit type --------------------------------
}  // extern "C"

namespace {
// Argument checks of the 16-bit-cache operator; *cap = the number of warp groups its workspace
// has room for (two slots of num_q_heads rows each).  A workspace too small for one group's
// slots -- the reference's [B, Hq, ceil(max / split)] sizing for a single short request -- still
// runs: with one group every sequence lies inside one chunk and nothing is written to it.
int validate_kv16(const pfd_decode_args* args, int* cap, int* sms_out, bool need_output) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu", args->struct_size,
                sizeof(pfd_decode_args));
  const pfd_decode_args& a = *args;
  if (a.batch < 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0) return fail(PFD_ERR_INVALID, "invalid query");
  if (a.head_dim != 128) return fail(PFD_ERR_UNSUPPORTED, "head_dim must be 128 for 16-bit caches");
  if (a.page_size != pfd::kPage) return fail(PFD_ERR_UNSUPPORTED, "page_size must be 16");
  if (a.num_q_heads % a.num_kv_heads != 0) return fail(PFD_ERR_INVALID, "Q heads must be divisible by KV heads");
  const int group = a.num_q_heads / a.num_kv_heads;
  if (group > 8) return fail(PFD_ERR_UNSUPPORTED, "at most 8 query heads per KV head for 16-bit caches");
  if (a.query_dtype != PFD_DTYPE_F16 && a.query_dtype != PFD_DTYPE_BF16)
    return fail(PFD_ERR_INVALID, "query must be FP16 or BF16");
  if (a.split_size < 16 || a.split_size % 16 != 0) return fail(PFD_ERR_INVALID, "split_size must be a multiple of 16");
  if (a.kv_start < 0 || a.max_seq_len < 0) return fail(PFD_ERR_INVALID, "negative length");
  *cap = 1;
  *sms_out = 0;
  if (a.batch == 0) return PFD_OK;
  if (a.batch > kChunkMaxBatch) return fail(PFD_ERR_UNSUPPORTED, "at most %d sequences per call", kChunkMaxBatch);
  if (!a.query || !a.key_cache || !a.value_cache || !a.block_table || !a.seq_lens)
    return fail(PFD_ERR_INVALID, "NULL operand");
  if (need_output && !a.output && !a.packed_output) return fail(PFD_ERR_INVALID, "no output given");
  if (a.q_stride_h % 2 || a.q_stride_b % 2 || (reinterpret_cast<uintptr_t>(a.query) & 3u))
    return fail(PFD_ERR_UNSUPPORTED, "query rows must be 4-byte aligned");
  if (!aligned16(a.key_cache) || !aligned16(a.value_cache) || a.k_stride_page % 8 || a.k_stride_token % 8 ||
      a.k_stride_head % 8 || a.v_stride_page % 8 || a.v_stride_token % 8 || a.v_stride_head % 8)
    return fail(PFD_ERR_UNSUPPORTED, "K/V cache base and strides must be multiples of 16 bytes");
  if (!(a.k_stride_page > 0 && a.v_stride_page > 0 && a.k_stride_token > 0 && a.v_stride_token > 0 &&
        a.k_stride_head > 0 && a.v_stride_head > 0 && a.num_pages > 0 &&
        head_is_dim1(a.k_stride_token, a.k_stride_head) == head_is_dim1(a.v_stride_token, a.v_stride_head)))
    return fail(PFD_ERR_UNSUPPORTED, "K and V caches must share one (page, token, head) order with positive strides");
  int64_t groups = 0;
  if (a.partial_output || a.partial_max || a.partial_sum) {
    if (!a.partial_output || !a.partial_max || !a.partial_sum)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape");
    if (a.partial_dtype < PFD_DTYPE_F32 || a.partial_dtype > PFD_DTYPE_BF16)
      return fail(PFD_ERR_INVALID, "partial_output dtype must be f32, f16 or bf16");
    if (!aligned16(a.partial_output)) return fail(PFD_ERR_UNSUPPORTED, "partial_output must be 16-byte aligned");
    if (a.partial_stride_s != 1 || a.partial_stride_h != a.workspace_splits ||
        a.partial_stride_b != (int64_t)a.num_q_heads * a.workspace_splits)
      return fail(PFD_ERR_UNSUPPORTED, "the partial workspace must be dense [batch, q heads, splits]");
    // The workspace is a flat list of rows, two slots of num_q_heads rows per group of warps: its
    // size caps the number of groups.
    const int64_t rows = (int64_t)a.batch * a.num_q_heads * a.workspace_splits;
    groups = rows / (2LL * a.num_q_heads);
  }
  if (int rc = enter_call()) return rc;
  *sms_out = t_device->sms;
  if (a.num_kv_heads > kChunkWarps16 * *sms_out / 2) return fail(PFD_ERR_UNSUPPORTED, "too many KV heads");
  *cap = (int)std::min<int64_t>(std::max<int64_t>(groups, 1), 1 << 20);
  return PFD_OK;
}
}  // namespace

extern "C" {

int pfd_paged_decode_kv16_split_out(const pfd_decode_args* args) {
  int cap = 1, sms = 0;
  if (int rc = validate_kv16(args, &cap, &sms, true)) return rc;
  const pfd_decode_args& a = *args;
  if (a.batch == 0) return PFD_OK;
  if (a.exchange != nullptr) return fail(PFD_ERR_UNSUPPORTED, "exchange: FP8 caches only");
  const int group = a.num_q_heads / a.num_kv_heads;
  const pfd::KernelParams kp = fill_params(a, group, !(a.flags & PFD_FLAG_NO_DIRECT_OUT), 0);
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  return a.query_dtype == PFD_DTYPE_BF16
             ? launch_balanced<true, kChunkStages16, kChunkWarps16, true>(a, kp, sms, stream, cap)
             : launch_balanced<false, kChunkStages16, kChunkWarps16, true>(a, kp, sms, stream, cap);
}

int64_t pfd_plan_bytes(int32_t batch, int32_t num_kv_heads) {
  if (batch < 0 || batch > kChunkMaxBatch || num_kv_heads <= 0)
    return fail(PFD_ERR_INVALID, "batch must be 0 .. %d and num_kv_heads positive", kChunkMaxBatch);
  if (int rc = enter_call()) return rc;
  const int sms = t_device->sms;
  const int max_groups = std::max(sms * kChunkWarps / num_kv_heads, 1);
  return 4 * pfd::plan_words(batch, max_groups, num_kv_heads);
}

int pfd_plan_decode(const pfd_decode_args* args, int32_t cache_elem_bytes, void* plan, int64_t plan_bytes) {
  if (plan == nullptr) return fail(PFD_ERR_INVALID, "plan is NULL");
  if (cache_elem_bytes != 1 && cache_elem_bytes != 2) return fail(PFD_ERR_INVALID, "cache_elem_bytes must be 1 or 2");
  if (reinterpret_cast<uintptr_t>(plan) & 15u) return fail(PFD_ERR_UNSUPPORTED, "plan must be 16-byte aligned");
  int num_warps = 0;
  if (cache_elem_bytes == 2) {
    int cap = 1, sms = 0;
    if (int rc = validate_kv16(args, &cap, &sms, false)) return rc;
    if (args->batch == 0) return PFD_OK;
    num_warps = balanced_num_warps(sms, kChunkWarps16, args->num_kv_heads, cap);
  } else {
    if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
    if (args->struct_size != sizeof(pfd_decode_args))
      return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu", args->struct_size,
                  sizeof(pfd_decode_args));
    const pfd_decode_args& a = *args;
    if (a.batch < 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0 || a.num_q_heads % a.num_kv_heads)
      return fail(PFD_ERR_INVALID, "invalid query");
    if (a.kv_start < 0) return fail(PFD_ERR_INVALID, "negative length");
    if (a.batch == 0) return PFD_OK;
    if (!a.block_table || !a.seq_lens) return fail(PFD_ERR_INVALID, "NULL operand");
    if (int rc = enter_call()) return rc;
    const int sms = t_device->sms;
    if (a.page_size != pfd::kPage || !balanced_eligible(a, a.num_q_heads / a.num_kv_heads, 0, sms))
      return fail(PFD_ERR_UNSUPPORTED,
                  "no plan: this call does not run the balanced kernel (head_dim 128, at most 8 query heads per KV "
                  "head, TMA-describable cache, dense f32 workspace of pfd_balanced_workspace_rows() rows, no "
                  "fixed-split flags)");
    num_warps = balanced_num_warps(sms, kChunkWarps, a.num_kv_heads, 0);
  }
  const pfd_decode_args& a = *args;
  const int max_groups = std::max(num_warps / a.num_kv_heads, 1);
  const int64_t need = 4 * pfd::plan_words(a.batch, max_groups, a.num_kv_heads);
  if (plan_bytes < need)
    return fail(PFD_ERR_INVALID, "plan buffer holds %lld bytes, this call needs %lld (pfd_plan_bytes)",
                (long long)plan_bytes, (long long)need);
  pfd::PlanParams pp{};
  pp.seq_lens = a.seq_lens;
  pp.block_table = a.block_table;
  pp.page_indptr = a.page_indptr;
  pp.bt_stride_b = a.bt_stride_b;
  pp.batch = a.batch;
  pp.kv_start = a.kv_start;
  pp.num_kv_heads = a.num_kv_heads;
  pp.max_groups = max_groups;
  pp.piece_cost = kChunkPieceCost;
  pp.plan = static_cast<int32_t*>(plan);
  const int ctas = std::max(1, std::min(8, (max_groups + 31) / 32));
  pfd::plan_decode_kernel<<<ctas, 1024, 0, static_cast<cudaStream_t>(a.stream)>>>(pp);
  return check_launch("plan kernel");
}

int pfd_shared_prefix_decode_fp8_e4m3(const pfd_decode_args* args, int32_t prefix_len) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu", args->struct_size,
                sizeof(pfd_decode_args));
  pfd_decode_args a = *args;
  if (a.head_dim != 128 || a.page_size != pfd::kPage)
    return fail(PFD_ERR_UNSUPPORTED, "the shared-prefix pass needs head_dim 128 and page_size 16");
  if (prefix_len <= 0 || prefix_len % pfd::kPage != 0 || prefix_len > a.max_seq_len)
    return fail(PFD_ERR_INVALID, "prefix_len must be a positive multiple of 16 not above max_seq_len");
  if (a.kv_start != 0) return fail(PFD_ERR_INVALID, "kv_start must be 0 for the shared-prefix pass");
  if (a.page_indptr != nullptr) return fail(PFD_ERR_UNSUPPORTED, "the shared-prefix pass needs a block table");
  if (a.batch <= 0) return a.batch == 0 ? PFD_OK : fail(PFD_ERR_INVALID, "invalid query");
  if (a.num_kv_heads <= 0 || a.num_q_heads % a.num_kv_heads != 0 || a.num_q_heads / a.num_kv_heads > 16)
    return fail(PFD_ERR_INVALID, "Q heads must be divisible by KV heads (at most 16 per KV head)");
  if (!a.partial_output || !a.partial_max || !a.partial_sum || a.partial_dtype != PFD_DTYPE_F32)
    return fail(PFD_ERR_INVALID, "the shared-prefix pass needs an f32 partial workspace");
  const int chunks = (prefix_len + pfd::kPrefixChunk - 1) / pfd::kPrefixChunk;
  if (!a.query || !a.key_cache || !a.value_cache || !a.block_table || !a.seq_lens)
    return fail(PFD_ERR_INVALID, "NULL operand");
  if ((reinterpret_cast<uintptr_t>(a.query) & 15u) || a.q_stride_h % 8 || a.q_stride_b % 8)
    return fail(PFD_ERR_UNSUPPORTED, "query rows must be 16-byte aligned for the shared-prefix pass");
  const bool bf16 = a.query_dtype == PFD_DTYPE_BF16;
  if (!bf16 && a.query_dtype != PFD_DTYPE_F16) return fail(PFD_ERR_INVALID, "query must be FP16 or BF16");
  // the suffix pass validates the rest (it sees the same operands) before anything is launched
  a.kv_start = prefix_len;
  a.flags |= PFD_FLAG_FIXED_SPLITS | PFD_FLAG_NO_DIRECT_OUT;
  a.flags &= ~(uint32_t)PFD_FLAG_PARTIAL_ONLY;
  a.plan = nullptr;
  if (a.exchange != nullptr) return fail(PFD_ERR_UNSUPPORTED, "exchange: not with the shared-prefix pass");
  {
    const int span = a.max_seq_len - prefix_len;
    const int ns = span > 0 ? (span + a.split_size - 1) / a.split_size : 1;
    if (a.split_size < 16 || a.split_size % 16) return fail(PFD_ERR_INVALID, "split_size must be a multiple of 16");
    if (a.workspace_splits < chunks + ns)
      return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape: the shared-prefix pass needs %d slots",
                  chunks + ns);
  }
  if (int rc = enter_call()) return rc;
  const int span = a.max_seq_len - prefix_len;
  const bool beside = suffix_beside_prefix(a, chunks, span > 0 ? (span + a.split_size - 1) / a.split_size : 1, false);
  if (int rc = bf16 ? launch_prefix<true>(a, prefix_len, chunks, beside) : launch_prefix<false>(a, prefix_len, chunks, beside))
    return rc;
  return decode_impl(&a, chunks);
}


// ---- allocation-free entry point -------------------------------------------------------
// The partial workspace of the split-KV path as a fixed array in the library image.  In host
// code the name below is only a stand-in for the symbol, never a device address: the address
// each device uses comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PFD_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

int pfd_shared_prefix_decode_grouped_fp8_e4m3(const pfd_decode_args* args, const void* groups, int32_t max_groups,
                                              int32_t max_prefix_len, int32_t max_suffix_len) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu", args->struct_size,
                sizeof(pfd_decode_args));
  pfd_decode_args a = *args;
  if (groups == nullptr || max_groups < 1) return fail(PFD_ERR_INVALID, "a groups buffer and its max_groups are needed");
  if (a.head_dim != 128 || a.page_size != pfd::kPage)
    return fail(PFD_ERR_UNSUPPORTED, "the shared-prefix pass needs head_dim 128 and page_size 16");
  if (max_prefix_len < 0 || max_suffix_len < 0) return fail(PFD_ERR_INVALID, "negative length");
  if (a.kv_start != 0) return fail(PFD_ERR_INVALID, "kv_start must be 0 for the shared-prefix pass");
  if (a.page_indptr != nullptr) return fail(PFD_ERR_UNSUPPORTED, "the shared-prefix pass needs a block table");
  if (a.exchange != nullptr) return fail(PFD_ERR_UNSUPPORTED, "exchange: not with the shared-prefix pass");
  if (a.batch <= 0) return a.batch == 0 ? PFD_OK : fail(PFD_ERR_INVALID, "invalid query");
  if (a.batch > pfd::kGroupsMaxBatch) return fail(PFD_ERR_UNSUPPORTED, "at most %d sequences per call", pfd::kGroupsMaxBatch);
  if (a.num_kv_heads <= 0 || a.num_q_heads % a.num_kv_heads != 0 || a.num_q_heads / a.num_kv_heads > 16)
    return fail(PFD_ERR_INVALID, "Q heads must be divisible by KV heads (at most 16 per KV head)");
  if (!a.partial_output || !a.partial_max || !a.partial_sum || a.partial_dtype != PFD_DTYPE_F32)
    return fail(PFD_ERR_INVALID, "the shared-prefix pass needs an f32 partial workspace");
  if (!a.query || !a.key_cache || !a.value_cache || !a.block_table || !a.seq_lens)
    return fail(PFD_ERR_INVALID, "NULL operand");
  if ((reinterpret_cast<uintptr_t>(a.query) & 15u) || a.q_stride_h % 8 || a.q_stride_b % 8)
    return fail(PFD_ERR_UNSUPPORTED, "query rows must be 16-byte aligned for the shared-prefix pass");
  const bool bf16 = a.query_dtype == PFD_DTYPE_BF16;
  if (!bf16 && a.query_dtype != PFD_DTYPE_F16) return fail(PFD_ERR_INVALID, "query must be FP16 or BF16");
  if (a.split_size < 16 || a.split_size % 16) return fail(PFD_ERR_INVALID, "split_size must be a multiple of 16");
  const int cap = std::min(max_prefix_len, a.max_seq_len) & ~15;  // no group's prefix pass reaches further
  const int chunks = (cap + pfd::kPrefixChunk - 1) / pfd::kPrefixChunk;
  // Requests in groups have at most max_suffix_len tokens behind their prefix (0 = unknown: the
  // whole context); a request in no group attends from 0 and gets the same number of splits, longer ones.
  const int suffix = max_suffix_len > 0 ? std::min(max_suffix_len, a.max_seq_len) : a.max_seq_len;
  const int ns = std::max((suffix + a.split_size - 1) / a.split_size, 1);
  const int split_loner = std::max(((a.max_seq_len + ns - 1) / ns + 15) / 16 * 16, a.split_size);
  if (a.workspace_splits < chunks + ns)
    return fail(PFD_ERR_INVALID, "partial output workspace has wrong shape: the grouped shared-prefix pass needs %d slots",
                chunks + ns);
  a.flags |= PFD_FLAG_FIXED_SPLITS | PFD_FLAG_NO_DIRECT_OUT;
  a.flags &= ~(uint32_t)PFD_FLAG_PARTIAL_ONLY;
  a.plan = nullptr;
  if (int rc = enter_call()) return rc;
  const int32_t* g = static_cast<const int32_t*>(groups);
  const bool beside = suffix_beside_prefix(a, chunks, ns, true);
  if (chunks > 0)
    if (int rc = bf16 ? launch_prefix<true>(a, cap, chunks, beside, g, max_groups)
                      : launch_prefix<false>(a, cap, chunks, beside, g, max_groups))
      return rc;
  GroupedRows rows;
  rows.row_kv_start = g + pfd::groups_row_prefix_off();
  rows.row_kv_cap = cap;
  rows.split_size_loner = split_loner;
  rows.num_splits = ns;
  return decode_impl(&a, chunks, &rows);
}

int pfd_paged_decode_fp8_e4m3_split_out_noalloc(const pfd_decode_args* args) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_decode_args))
    return fail(PFD_ERR_INVALID, "pfd_decode_args size mismatch: caller %u, library %zu",
                args->struct_size, sizeof(pfd_decode_args));
  pfd_decode_args a = *args;
  if (a.batch < 0 || a.num_q_heads <= 0 || a.head_dim <= 0 || a.split_size < 16 || a.kv_start < 0 ||
      a.max_seq_len < 0)
    return fail(PFD_ERR_INVALID, "invalid geometry");
  if (a.page_indptr != nullptr)
    return fail(PFD_ERR_UNSUPPORTED,
                "the allocation-free entry point takes a block table: page_indptr addressing needs the balanced "
                "kernel, which this entry point never runs");
  if (a.flags & PFD_FLAG_PARTIAL_ONLY)
    return fail(PFD_ERR_UNSUPPORTED,
                "PFD_FLAG_PARTIAL_ONLY makes no sense here: the partials would stay in the library's own array");
  a.plan = nullptr;
  if (a.exchange != nullptr) return fail(PFD_ERR_UNSUPPORTED, "exchange: not with the allocation-free entry point");
  const int64_t span = a.max_seq_len > a.kv_start ? a.max_seq_len - a.kv_start : 0;
  int64_t splits = (span + a.split_size - 1) / a.split_size;
  if (splits < 1) splits = 1;
  const int64_t rows = (int64_t)a.batch * a.num_q_heads * splits;
  const int64_t need = rows * (a.head_dim + 2) * (int64_t)sizeof(float);
  // With a single split every work item writes its final rows itself and the array is not touched.
  const bool touches_scratch = splits > 1 || (a.flags & PFD_FLAG_NO_DIRECT_OUT);
  if (touches_scratch && need > (int64_t)PFD_NOALLOC_SCRATCH_BYTES)
    return fail(PFD_ERR_UNSUPPORTED,
                "request needs %lld bytes of split-KV scratch but the built-in array holds %u; "
                "raise split_size or use the entry point that takes a workspace",
                (long long)need, PFD_NOALLOC_SCRATCH_BYTES);
  if (!touches_scratch) {  // no partials: run as the ordinary entry point does without a workspace
    a.partial_output = nullptr;
    a.partial_max = a.partial_sum = nullptr;
    a.workspace_splits = 0;
    a.flags |= PFD_FLAG_FIXED_SPLITS;
    return pfd_paged_decode_fp8_e4m3_split_out(&a);
  }
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
  a.flags |= PFD_FLAG_FIXED_SPLITS;  // the array is sized for split_size-sized splits
  return pfd_paged_decode_fp8_e4m3_split_out(&a);
}

int pfd_rope_quant_append(const pfd_rope_args* args) {
  if (args == nullptr) return fail(PFD_ERR_INVALID, "args is NULL");
  if (args->struct_size != sizeof(pfd_rope_args))
    return fail(PFD_ERR_INVALID, "pfd_rope_args size mismatch: caller %u, library %zu", args->struct_size,
                sizeof(pfd_rope_args));
  const pfd_rope_args& a = *args;
  if (a.num_tokens < 0 || a.num_q_heads <= 0 || a.num_kv_heads <= 0 || a.head_dim <= 0 || a.block_size <= 0)
    return fail(PFD_ERR_INVALID, "invalid geometry");
  if (a.query_dtype != PFD_DTYPE_F16 && a.query_dtype != PFD_DTYPE_BF16)
    return fail(PFD_ERR_INVALID, "query must be FP16 or BF16");
  if (a.rotary_dim <= 0 || a.rotary_dim > a.head_dim || a.rotary_dim % 2)
    return fail(PFD_ERR_INVALID, "invalid cos_sin_cache rotary dimension");
  if (a.cos_sin_dtype != PFD_DTYPE_F32 && a.cos_sin_dtype != a.query_dtype)
    return fail(PFD_ERR_INVALID, "cos_sin_cache must be float32 or have the query's dtype");
  if (a.cache_dtype != PFD_DTYPE_E4M3 && a.cache_dtype != a.query_dtype)
    return fail(PFD_ERR_INVALID, "the caches must be FP8-e4m3 or have the query's dtype");
  if (a.num_tokens == 0) return PFD_OK;
  if (!a.query || !a.key || !a.value || !a.positions || !a.cos_sin_cache || !a.slot_mapping || !a.key_cache ||
      !a.value_cache)
    return fail(PFD_ERR_INVALID, "NULL operand");
  if (a.cache_dtype == PFD_DTYPE_E4M3 &&
      ((!a.k_scale_per_head && !(a.k_scale > 0.f)) || (!a.v_scale_per_head && !(a.v_scale > 0.f))))
    return fail(PFD_ERR_INVALID, "FP8 caches need positive scales");
  pfd::RopeParams p{};
  p.query = a.query; p.key = a.key; p.value = a.value;
  p.positions = a.positions; p.cos_sin_cache = a.cos_sin_cache; p.slot_mapping = a.slot_mapping;
  p.key_cache = a.key_cache; p.value_cache = a.value_cache;
  p.k_scale_ph = a.k_scale_per_head; p.v_scale_ph = a.v_scale_per_head;
  p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  p.q_stride_t = a.q_stride_t; p.q_stride_h = a.q_stride_h;
  p.k_stride_t = a.k_stride_t; p.k_stride_h = a.k_stride_h;
  p.v_stride_t = a.v_stride_t; p.v_stride_h = a.v_stride_h;
  p.kc_stride_block = a.kc_stride_block; p.kc_stride_token = a.kc_stride_token; p.kc_stride_head = a.kc_stride_head;
  p.vc_stride_block = a.vc_stride_block; p.vc_stride_token = a.vc_stride_token; p.vc_stride_head = a.vc_stride_head;
  p.cs_stride = a.cos_sin_stride;
  p.num_tokens = a.num_tokens; p.num_q_heads = a.num_q_heads; p.num_kv_heads = a.num_kv_heads;
  p.head_dim = a.head_dim; p.rotary_dim = a.rotary_dim; p.block_size = a.block_size;
  p.is_neox = a.is_neox ? 1 : 0;
  p.cos_sin_f32 = a.cos_sin_dtype == PFD_DTYPE_F32 ? 1 : 0;
  p.cache_fp8 = a.cache_dtype == PFD_DTYPE_E4M3 ? 1 : 0;
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  // The vectorised kernel: NeoX pairs over the whole head, rows and caches 16-byte aligned.
  const auto al = [](const void* ptr, int64_t bytes) { return (reinterpret_cast<uintptr_t>(ptr) & (uintptr_t)(bytes - 1)) == 0; };
  const auto m8 = [](int64_t x) { return x % 8 == 0; };
  const int cache_elem = p.cache_fp8 ? 1 : 2;
  const bool vec = p.is_neox && a.rotary_dim == a.head_dim && a.head_dim % 16 == 0 &&
                   al(a.query, 16) && al(a.key, 16) && al(a.value, 16) && al(a.cos_sin_cache, 16) &&
                   m8(a.q_stride_t) && m8(a.q_stride_h) && m8(a.k_stride_t) && m8(a.k_stride_h) && m8(a.v_stride_t) &&
                   m8(a.v_stride_h) && (p.cos_sin_f32 ? a.cos_sin_stride % 4 == 0 : m8(a.cos_sin_stride)) &&
                   al(a.key_cache, 8 * cache_elem) && al(a.value_cache, 8 * cache_elem) && m8(a.kc_stride_block) &&
                   m8(a.kc_stride_token) && m8(a.kc_stride_head) && m8(a.vc_stride_block) && m8(a.vc_stride_token) &&
                   m8(a.vc_stride_head);
  if (vec) {
    if (a.query_dtype == PFD_DTYPE_BF16) pfd::rope_quant_append_vec_kernel<true><<<a.num_tokens, 256, 0, stream>>>(p);
    else pfd::rope_quant_append_vec_kernel<false><<<a.num_tokens, 256, 0, stream>>>(p);
    return check_launch("rope + append kernel (vectorised)");
  }
  if (a.query_dtype == PFD_DTYPE_BF16) pfd::rope_quant_append_kernel<true><<<a.num_tokens, 256, 0, stream>>>(p);
  else pfd::rope_quant_append_kernel<false><<<a.num_tokens, 256, 0, stream>>>(p);
  return check_launch("rope + append kernel");
}

int pfd_last_path(void) { return g_last_path; }

int64_t pfd_balanced_workspace_rows(int32_t num_q_heads, int32_t num_kv_heads) {
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads)
    return fail(PFD_ERR_INVALID, "Q heads must be divisible by KV heads");
  if (int rc = enter_call()) return rc;
  const int sms = t_device->sms;
  return 2LL * (sms * kChunkWarps / num_kv_heads) * num_q_heads;
}

#ifdef PFD_PHASE_STAMPS
// Tuning builds only: while `device_buffer` (uint64 [slots][8], caller-owned device memory) is
// set, the kernels store %globaltimer stamps of their phases there.  Not part of the shipped ABI.
int pfd_debug_phase_times(void* device_buffer) {
  g_phase_times = static_cast<unsigned long long*>(device_buffer);
  cudaMemcpyToSymbol(pfd::g_dbg_stamps, &g_phase_times, sizeof g_phase_times);
  return PFD_OK;
}
#endif

int pfd_set_suffix_form(int32_t form) {
  if (form < -1 || form > 1) return fail(PFD_ERR_INVALID, "form must be -1, 0 or 1");
  g_suffix_form.store(form, std::memory_order_relaxed);
  return PFD_OK;
}

int pfd_set_wait_limit_ns(uint64_t limit_ns) {
  if (limit_ns == 0) return fail(PFD_ERR_INVALID, "the wait limit must be positive");
  g_wait_limit_ns.store(limit_ns, std::memory_order_relaxed);
  return PFD_OK;
}

int pfd_selftest_bounded_wait(uint64_t limit_ns, uint64_t* waited_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000ull * 1000 * 1000)
    return fail(PFD_ERR_INVALID, "limit_ns must be between 1 ns and 1 s");
  if (int rc = enter_call()) return rc;
  int32_t* status = nullptr;
  if (int rc = status_pointer(&status)) return rc;
  unsigned long long* dev_waited = nullptr;
  // the word behind the status word of the same symbol would need a second symbol: keep the
  // result in mapped pinned host memory instead, which needs no device allocation
  unsigned long long* host_waited = nullptr;
  if (waited_ns != nullptr) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&host_waited), sizeof(unsigned long long), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_waited), host_waited, 0) != cudaSuccess) {
      if (host_waited) cudaFreeHost(host_waited);
      return fail(PFD_ERR_CUDA, "pinned host memory for the self-test is not available");
    }
    *host_waited = 0;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  pfd::bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_ns, dev_waited);
  int rc = check_launch("bounded-wait self-test kernel");
  if (rc == PFD_OK && cudaStreamSynchronize(s) != cudaSuccess) rc = fail(PFD_ERR_CUDA, "the self-test kernel failed");
  if (waited_ns != nullptr) {
    *waited_ns = *host_waited;
    cudaFreeHost(host_waited);
  }
  return rc;
}

int pfd_device_status(int32_t* status) {
  if (status == nullptr) return fail(PFD_ERR_INVALID, "status is NULL");
  if (int rc = enter_call()) return rc;
  int32_t* p = nullptr;
  if (int rc = status_pointer(&p)) return rc;
  cudaError_t e = cudaDeviceSynchronize();  // kernels on non-blocking streams included
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaDeviceSynchronize failed: %s", cudaGetErrorString(e));
  e = cudaMemcpy(status, p, sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "reading the device status failed: %s", cudaGetErrorString(e));
  if (*status != 0) {
    const int32_t zero = 0;
    e = cudaMemcpy(p, &zero, sizeof(int32_t), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "clearing the device status failed: %s", cudaGetErrorString(e));
  }
  return PFD_OK;
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

int64_t pfd_exchange_control_offset(int32_t world, int64_t rows, int32_t head_dim) {
  if (world < 1 || world > 8 || rows < 0 || head_dim != 128) return fail(PFD_ERR_INVALID, "invalid exchange geometry");
  static_assert(PFD_XCH_ROW == pfd::kXchRow, "row layout");
  const int64_t recv = 2LL * world * rows * PFD_XCH_ROW * 8;
  return (recv + 255) / 256 * 256;
}

int64_t pfd_exchange_bytes(int32_t world, int64_t rows, int32_t head_dim) {
  const int64_t off = pfd_exchange_control_offset(world, rows, head_dim);
  return off < 0 ? off : off + 256;
}

int pfd_exchange_alloc(int64_t bytes, void** ptr, pfd_ipc_handle* handle) {
  if (bytes <= 0 || ptr == nullptr || handle == nullptr) return fail(PFD_ERR_INVALID, "invalid argument");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaMalloc of the exchange buffer failed: %s", cudaGetErrorString(e));
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(PFD_ERR_CUDA, "preparing the exchange buffer failed: %s", cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(pfd_ipc_handle), "IPC handle size");
  memcpy(handle->bytes, &h, sizeof h);
  *ptr = p;
  return PFD_OK;
}

int pfd_exchange_open(const pfd_ipc_handle* handle, void** peer_ptr) {
  if (handle == nullptr || peer_ptr == nullptr) return fail(PFD_ERR_INVALID, "invalid argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle->bytes, sizeof h);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  *peer_ptr = p;
  return PFD_OK;
}

int pfd_exchange_close(void* peer_ptr) {
  if (peer_ptr == nullptr) return PFD_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  return e == cudaSuccess ? PFD_OK : fail(PFD_ERR_CUDA, "cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
}

int pfd_exchange_free(void* ptr) {
  if (ptr == nullptr) return PFD_OK;
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? PFD_OK : fail(PFD_ERR_CUDA, "cudaFree failed: %s", cudaGetErrorString(e));
}

int pfd_exchange_merge(const pfd_exchange* exchange, int64_t rows, int32_t head_dim, void* output,
                       int32_t out_dtype, void* stream) {
  if (exchange == nullptr || output == nullptr) return fail(PFD_ERR_INVALID, "NULL operand");
  const pfd_exchange& x = *exchange;
  if (x.world < 1 || x.world > 8 || x.rank < 0 || x.rank >= x.world || !x.control)
    return fail(PFD_ERR_INVALID, "exchange: world 1..8, 0 <= rank < world and the control words are needed");
  if (!x.recv[x.rank]) return fail(PFD_ERR_INVALID, "exchange: this rank's recv pointer is NULL");
  if (head_dim != 128) return fail(PFD_ERR_UNSUPPORTED, "exchange: head_dim must be 128");
  if (out_dtype < PFD_DTYPE_F32 || out_dtype > PFD_DTYPE_BF16)
    return fail(PFD_ERR_INVALID, "output dtype must be f32, f16 or bf16");
  if (rows <= 0) return rows == 0 ? PFD_OK : fail(PFD_ERR_INVALID, "negative row count");
  if (int rc = enter_call()) return rc;
  pfd::TmaParams tp{};
  if (int rc = status_pointer(&tp.status)) return rc;
  tp.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  tp.phase_times = g_phase_times;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((rows + 3) / 4));
  cfg.blockDim = dim3(128);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const unsigned long long* recv = static_cast<const unsigned long long*>(x.recv[x.rank]);
  uint32_t* control = static_cast<uint32_t*>(x.control);
  const int world = x.world;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, pfd::exchange_merge_kernel<128>, recv, control, world, rows,
                                           output, (int)out_dtype, tp);
  if (e != cudaSuccess) return fail(PFD_ERR_CUDA, "exchange merge kernel launch failed: %s", cudaGetErrorString(e));
  return check_launch("exchange merge kernel");
}

int64_t pfd_prefix_groups_bytes(int32_t batch, int32_t max_groups) {
  if (batch < 0 || batch > pfd::kGroupsMaxBatch || max_groups < 1)
    return fail(PFD_ERR_INVALID, "batch must be 0 .. %d and max_groups positive", pfd::kGroupsMaxBatch);
  return 4 * pfd::groups_words(batch, max_groups);
}

int pfd_group_shared_prefixes(const int32_t* block_table, int64_t bt_stride_b, int32_t bt_cols,
                              const int32_t* prefix_lengths, int32_t uniform_prefix_len, const int32_t* seq_lens,
                              int32_t batch, int32_t min_batch, int32_t min_prefix_len, int32_t max_groups,
                              void* groups, int64_t groups_bytes, void* stream) {
  if (batch < 0 || batch > pfd::kGroupsMaxBatch)
    return fail(PFD_ERR_UNSUPPORTED, "at most %d sequences per call", pfd::kGroupsMaxBatch);
  if (min_batch < 1 || min_prefix_len < 0 || max_groups < 1 || bt_cols < 0 || uniform_prefix_len < 0)
    return fail(PFD_ERR_INVALID, "min_batch and max_groups must be positive, lengths non-negative");
  if (groups == nullptr || groups_bytes < 4 * pfd::groups_words(batch, max_groups))
    return fail(PFD_ERR_INVALID, "groups buffer holds %lld bytes, this call needs %lld (pfd_prefix_groups_bytes)",
                (long long)groups_bytes, (long long)(4 * pfd::groups_words(batch, max_groups)));
  if (batch > 0 && block_table == nullptr) return fail(PFD_ERR_INVALID, "NULL operand");
  if (prefix_lengths == nullptr && uniform_prefix_len == 0 && seq_lens == nullptr)
    return fail(PFD_ERR_INVALID, "give prefix_lengths, a uniform prefix length, or seq_lens to derive one from");
  pfd::GroupParams gp{};
  gp.block_table = block_table;
  gp.bt_stride_b = bt_stride_b;
  gp.bt_cols = bt_cols;
  gp.prefix_lengths = prefix_lengths;
  gp.uniform_prefix_len = uniform_prefix_len;
  gp.seq_lens = seq_lens;
  gp.batch = batch;
  gp.min_batch = min_batch;
  gp.min_prefix_len = min_prefix_len;
  gp.max_groups = max_groups;
  gp.groups = static_cast<int32_t*>(groups);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (batch > 0) {
    pfd::prefix_hash_kernel<<<batch, 256, 0, s>>>(gp);
    if (int rc = check_launch("prefix hash kernel")) return rc;
    pfd::prefix_match_kernel<<<batch, 256, 0, s>>>(gp);
    if (int rc = check_launch("prefix match kernel")) return rc;
  }
  pfd::prefix_finish_kernel<<<1, 1024, 0, s>>>(gp);
  return check_launch("prefix finish kernel");
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
