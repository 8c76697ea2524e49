// mb_gemm_u8_static_scratch: the tensor-core uint8 GEMM for callers that must
// not allocate.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a
// real-time inference loop that has promised its host a fixed memory
// footprint, inside a plugin whose embedding application owns all device
// memory, or in a callback that may run while another stream is being
// captured (an allocation there would break the capture).  mb_gemm_u8 keeps
// its operand byte sums in a growable arena and needs an mb_context, both of
// which come from cudaMalloc.  This variant needs neither: its scratch is a
// fixed array that is part of the library image.
//
// The price: one array per GPU for the life of the process (130 KB on every
// GPU that loads the library), a size limit (M, N <= 16384, one batch entry),
// and no concurrency -- every call on a device uses the same array, so two
// calls whose kernels overlap on the GPU (different streams, or different
// host threads) race on it.  Issue calls on one stream, or order them with
// events.
#include <mutex>

#include "common.cuh"

bool mb_gemm_u8_tc_supported(const mb_context *ctx, const void *A, const void *B, int64_t M,
                             int64_t N, int64_t K, bool a_mn, bool b_mn, int a_batched,
                             int b_batched);
int mb_gemm_u8_tc_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                         const uint32_t *sum_a, const uint32_t *sum_b, const int32_t *bias,
                         void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                         int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                         int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                         int bias_per_row);

namespace {

constexpr int64_t kMaxDim = MB_STATIC_SCRATCH_MAX_DIM;

// [0, kMaxDim)            byte sums of the rows of A
// [kMaxDim, 2 kMaxDim)    byte sums of the columns of B
// [2 kMaxDim]             status word of the GEMM kernel's bounded waits
// In host code this name is only a handle for cudaGetSymbolAddress; it is not
// a device address and must never be passed to a kernel.
static __device__ __align__(256) uint32_t g_static_scratch[2 * kMaxDim + 64];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
uint32_t *g_scratch_addr[kMaxDevices] = {nullptr};  // device address per GPU
int g_num_sms[kMaxDevices] = {0};
// kernels whose shared-memory limit was already raised on each GPU (the launcher sets the
// attribute once per device and kernel variant and records it in its context; the per-call
// context view below carries this mask in and out so that later calls skip the attribute call)
uint64_t g_func_attr_mask[kMaxDevices] = {0};
void *g_encode_tiled = nullptr;

// Sum of each row of a [rows x len] byte matrix (len % 16 == 0): one warp per
// row.  Overwrites its outputs, so nothing needs clearing first.
__global__ void __launch_bounds__(256) static_rowsum_kernel(const uint8_t *__restrict__ x,
                                                            int64_t rows, int64_t len,
                                                            int out_offset) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint4 *p = reinterpret_cast<const uint4 *>(x + row * len);
  uint32_t s = 0;
  for (int64_t i = lane; i < (len >> 4); i += 32) {
    const uint4 v = __ldg(p + i);
    s = __dp4a(v.x, 0x01010101u, s);
    s = __dp4a(v.y, 0x01010101u, s);
    s = __dp4a(v.z, 0x01010101u, s);
    s = __dp4a(v.w, 0x01010101u, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) g_static_scratch[out_offset + row] = s;  // device code may name the array
}

// Sum down the columns of a [rows x cols] byte matrix (cols % 4 == 0): each
// thread owns 4 adjacent columns and walks all rows, so it too overwrites its
// outputs and leaves nothing of the previous call behind.
__global__ void __launch_bounds__(128) static_colsum_kernel(const uint8_t *__restrict__ x,
                                                            int64_t rows, int64_t cols,
                                                            int out_offset) {
  const int64_t c4 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c4 * 4 >= cols) return;
  uint32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  for (int64_t r = 0; r < rows; ++r) {
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(x + r * cols) + c4);
    s0 += w & 0xffu;
    s1 += (w >> 8) & 0xffu;
    s2 += (w >> 16) & 0xffu;
    s3 += w >> 24;
  }
  uint32_t *o = g_static_scratch + out_offset + c4 * 4;
  o[0] = s0; o[1] = s1; o[2] = s2; o[3] = s3;
}

// Once per device, with that device current: ask the runtime where the array
// lives on this GPU.  No allocation happens here; the array came with the
// module.
int setup_device(int device, char *err, size_t err_len) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[device] != nullptr) return MB_SUCCESS;
  void *ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess) {
    snprintf(err, err_len, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    return MB_RUNTIME_ERROR;
  }
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess || sms <= 0) {
    snprintf(err, err_len, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    return MB_RUNTIME_ERROR;
  }
  if (g_encode_tiled == nullptr) {
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      snprintf(err, err_len, "cuTensorMapEncodeTiled is not available");
      return MB_RUNTIME_ERROR;
    }
    g_encode_tiled = fn;
  }
  g_num_sms[device] = sms;
  g_scratch_addr[device] = static_cast<uint32_t *>(ptr);
  return MB_SUCCESS;
}

}  // namespace

extern "C" int mb_gemm_u8_static_scratch(void *stream, const uint8_t *A, const uint8_t *B,
                                         const int32_t *bias, void *C, int out_is_int32,
                                         int64_t M, int64_t N, int64_t K, int a_col_major,
                                         int b_col_major, int32_t zp_a, int32_t zp_b,
                                         int32_t multiplier, int32_t right_shift,
                                         int32_t zp_c, int bias_per_row, char *error_message,
                                         size_t error_message_len) {
  char local_err[8];
  char *err = error_message != nullptr ? error_message : local_err;
  const size_t err_len = error_message != nullptr ? error_message_len : sizeof(local_err);
  if (err_len > 0) err[0] = 0;
  if (M < 0 || N < 0 || K < 1) {
    snprintf(err, err_len, "bad dimension M=%lld N=%lld K=%lld", (long long)M, (long long)N,
             (long long)K);
    return MB_INVALID_ARGS;
  }
  if (M == 0 || N == 0) return MB_SUCCESS;
  if (M > kMaxDim || N > kMaxDim) {
    snprintf(err, err_len,
             "M=%lld, N=%lld exceed the static scratch limit of %lld per dimension; "
             "use mb_gemm_u8 (which allocates) for larger problems",
             (long long)M, (long long)N, (long long)kMaxDim);
    return MB_INVALID_ARGS;
  }
  if (A == nullptr || B == nullptr || C == nullptr) {
    snprintf(err, err_len, "null operand");
    return MB_INVALID_ARGS;
  }
  if (!out_is_int32 && (multiplier <= 0 || right_shift < 0 || right_shift > 31)) {
    snprintf(err, err_len, "bad multiplier %d / shift %d", multiplier, right_shift);
    return MB_INVALID_ARGS;
  }
  if (!out_is_int32 && (zp_c < 0 || zp_c > 255)) {
    snprintf(err, err_len, "output zero point %d outside uint8", zp_c);
    return MB_INVALID_ARGS;
  }
  if (zp_a < 0 || zp_a > 255 || zp_b < 0 || zp_b > 255) {
    snprintf(err, err_len, "operand zero points %d / %d outside uint8", zp_a, zp_b);
    return MB_INVALID_ARGS;
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    snprintf(err, err_len, "no current CUDA device");
    return MB_RUNTIME_ERROR;
  }
  int st = setup_device(device, err, err_len);
  if (st != MB_SUCCESS) return st;
  uint32_t *scratch = g_scratch_addr[device];

  // A view of the launcher's context that lives on this stack frame: the
  // stream, the SM count, and the status word inside the static array.
  mb_context view;
  view.device = device;
  view.num_sms = g_num_sms[device];
  view.stream = static_cast<cudaStream_t>(stream);
  view.encode_tiled = g_encode_tiled;
  view.dev_status = reinterpret_cast<int *>(scratch + 2 * kMaxDim);
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    view.func_attr_mask = g_func_attr_mask[device];
  }

  const bool a_mn = a_col_major != 0, b_mn = b_col_major == 0;
  if (!mb_gemm_u8_tc_supported(&view, A, B, M, N, K, a_mn, b_mn, 0, 0) || K % 16 != 0) {
    snprintf(err, err_len,
             "operands must be 16-byte aligned with K and the contiguous dimension of each "
             "operand a multiple of 16 (and K <= 33000)");
    return MB_UNSUPPORTED;
  }
  // Every call starts from a clean status word; the sums are overwritten in
  // full by the kernels below, so stale values of an earlier, larger problem
  // are never read.
  cudaError_t e = cudaMemsetAsync(view.dev_status, 0, sizeof(int), view.stream);
  if (e == cudaSuccess && zp_b != 0) {
    if (a_mn)
      static_colsum_kernel<<<static_cast<unsigned>(ceil_div64(ceil_div64(M, 4), 128)), 128, 0,
                             view.stream>>>(A, K, M, 0);
    else
      static_rowsum_kernel<<<static_cast<unsigned>(ceil_div64(M, 8)), 256, 0, view.stream>>>(
          A, M, K, 0);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess && zp_a != 0) {
    if (b_mn)
      static_colsum_kernel<<<static_cast<unsigned>(ceil_div64(ceil_div64(N, 4), 128)), 128, 0,
                             view.stream>>>(B, K, N, static_cast<int>(kMaxDim));
    else
      static_rowsum_kernel<<<static_cast<unsigned>(ceil_div64(N, 8)), 256, 0, view.stream>>>(
          B, N, K, static_cast<int>(kMaxDim));
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    snprintf(err, err_len, "sum kernels: %s", cudaGetErrorString(e));
    return MB_RUNTIME_ERROR;
  }
  st = mb_gemm_u8_tc_launch(&view, A, B, zp_b != 0 ? scratch : nullptr,
                            zp_a != 0 ? scratch + kMaxDim : nullptr, bias, C, out_is_int32, 1, M,
                            N, K, a_mn, b_mn, 0, 0, zp_a, zp_b, multiplier, right_shift, zp_c,
                            bias_per_row);
  if (st != MB_SUCCESS) snprintf(err, err_len, "%s", view.last_error);
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    g_func_attr_mask[device] |= view.func_attr_mask;
  }
  return st;
}

// The GEMM kernel bounds every wait on a barrier; when one runs out it writes a non-zero code
// into its status word, stops, and leaves C partly written.  mb_gemm_u8 reports that through
// mb_stream_sync; this entry point has no context to sync, so the caller asks here: the word
// of the LAST call on the current device is copied into *host_status by an asynchronous copy
// on `stream` (no allocation; pinned memory makes it truly asynchronous).  After the stream
// has been synchronized, 0 means the last call ran to completion.
extern "C" int mb_gemm_u8_static_scratch_status(void *stream, int *host_status) {
  if (host_status == nullptr) return MB_INVALID_ARGS;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return MB_RUNTIME_ERROR;
  const uint32_t *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    scratch = g_scratch_addr[device];
  }
  if (scratch == nullptr) {  // no call has run on this device yet
    *host_status = 0;
    return MB_SUCCESS;
  }
  const cudaError_t e = cudaMemcpyAsync(host_status, scratch + 2 * kMaxDim, sizeof(int),
                                        cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MB_SUCCESS : MB_RUNTIME_ERROR;
}
