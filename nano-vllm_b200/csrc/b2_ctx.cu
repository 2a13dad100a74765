// Context: symmetric buffers shared between tensor-parallel ranks through CUDA
// IPC, rank-local scratch, the host-visible status word, and the TMA
// descriptor encoder.
#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "b2_common.cuh"

namespace {
thread_local char g_last_error[512] = "";
std::atomic<int64_t> g_launches{0};

// cuTensorMapEncodeTiled, fetched through the runtime so that the library does
// not link against libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

__global__ void b2_fill_u32_kernel(uint32_t* p, size_t n, uint32_t v) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) p[i] = v;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
}  // namespace

namespace b2 {
int set_cuda_error(cudaError_t e, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return B2_ERR_CUDA;
}
int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("B2_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t ld_elems,
                   uint32_t box_inner, uint32_t box_rows) {
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (fn == nullptr || q != cudaDriverEntryPointSuccess) {
      snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled not available from the driver");
      return B2_ERR_CUDA;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {ld_elems * 2};  // bytes between rows
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error),
             "cuTensorMapEncodeTiled failed (%d): base=%p inner=%llu rows=%llu ld=%llu box=%ux%u", static_cast<int>(r), base,
             static_cast<unsigned long long>(inner), static_cast<unsigned long long>(rows),
             static_cast<unsigned long long>(ld_elems), box_inner, box_rows);
    return B2_ERR_CUDA;
  }
  return B2_OK;
}
}  // namespace b2

extern "C" {

const char* b2_last_error(void) { return g_last_error; }
int64_t b2_launch_count(void) { return g_launches.load(); }

static int ctx_init(b2_ctx* c);

// Data-as-flag buffers start out "not written" (the sentinel), flags and counters at zero, the token inbox at -1.
static int init_symmetric_region(b2_ctx* c) {
  const size_t words = c->off_logits / 4;
  b2_fill_u32_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(c->symm), words, B2_SENTINEL32);
  b2::count_launch();
  B2_CUDA(cudaGetLastError());
  B2_CUDA(cudaMemset(c->symm + c->off_logits, 0, c->off_tokens - c->off_logits));
  B2_CUDA(cudaMemset(c->symm + c->off_tokens, 0xFF, c->symm_bytes - c->off_tokens));
  return B2_OK;
}

int b2_ctx_create(const b2_config* cfg, b2_ctx** out) {
  if (cfg == nullptr || out == nullptr) return B2_ERR_ARG;
  *out = nullptr;
  if (cfg->world < 1 || cfg->world > B2_MAX_WORLD || cfg->rank < 0 || cfg->rank >= cfg->world) return B2_ERR_ARG;
  if (cfg->max_tokens < 1 || cfg->hidden < 8 || cfg->hidden % 8 != 0) return B2_ERR_ARG;
  b2_ctx* c = new (std::nothrow) b2_ctx();
  if (c == nullptr) return B2_ERR_ARG;
  memset(c, 0, sizeof(*c));
  c->cfg = *cfg;
  if (c->cfg.oneshot_tokens <= 0) c->cfg.oneshot_tokens = 1024;
  if (c->cfg.oneshot_tokens > c->cfg.max_tokens) c->cfg.oneshot_tokens = c->cfg.max_tokens;
  if (c->cfg.timeout_ms <= 0) c->cfg.timeout_ms = 5000;
  c->rowpar_form = B2_FORM_AUTO;
  c->owner_min_tokens = 65;
  // measured at Qwen3-32B shapes: the two-shot form takes over at 1024 tokens at 8 ranks and at 512 at 4 ranks; at 2 ranks
  // the one-shot form (one copy either way) stays ahead up to its buffer's size
  c->owner_max_tokens = std::min(c->cfg.world >= 8 ? 1023 : 511, c->cfg.oneshot_tokens);
  c->twoshot_min_tokens = c->cfg.world >= 4 ? c->owner_max_tokens + 1 : std::min(1024, c->cfg.oneshot_tokens) + 1;
  c->whole_tiles = true;
  const int rc = ctx_init(c);
  if (rc != B2_OK) {
    b2_ctx_destroy(c);  // frees whatever was allocated before the failing call; the error text stays
    return rc;
  }
  *out = c;
  return B2_OK;
}

static int ctx_init(b2_ctx* c) {
  const b2_config* cfg = &c->cfg;
  B2_CUDA(cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  B2_CUDA(cudaGetDeviceProperties(&prop, cfg->device));
  c->num_sms = prop.multiProcessorCount;

  // ---- symmetric region ----------------------------------------------------
  const size_t W = static_cast<size_t>(c->cfg.world), H = static_cast<size_t>(c->cfg.hidden);
  size_t off = 0;
  c->off_rowpar = off;
  off = align_up(off + 2 * W * c->cfg.oneshot_tokens * H * 2, 1024);
  c->off_embed = off;
  if (W > 1) off = align_up(off + 2 * static_cast<size_t>(c->cfg.max_tokens) * H * 2, 1024);
  c->off_inbox2 = off;
  const size_t rows_per_rank = ((static_cast<size_t>(c->cfg.max_tokens) + 15) / 16 + W - 1) / W * 16;  // 16-row blocks dealt round-robin
  if (W > 1) off = align_up(off + 2 * W * rows_per_rank * H * 2, 1024);
  // owner form of the fused row-parallel block (few tokens): owners' inbox and every rank's landing buffer
  c->off_inbox3 = off;
  const size_t rows3 = (static_cast<size_t>(c->cfg.oneshot_tokens) + W - 1) / W;
  off = align_up(off + 2 * W * rows3 * H * 2, 1024);
  c->off_land = off;
  off = align_up(off + 2 * 2 * static_cast<size_t>(c->cfg.oneshot_tokens) * H * 2, 1024);
  c->off_logits = off;  // everything below this offset is a data-as-flag buffer (starts out holding the sentinel)
  if (c->cfg.vocab > 0 && c->cfg.max_seqs > 0) off = align_up(off + static_cast<size_t>(c->cfg.max_seqs) * c->cfg.vocab * 2, 1024);
  c->off_flags = off;
  off = align_up(off + 256, 1024);
  c->off_out = off;
  if (W > 1) off = align_up(off + static_cast<size_t>(c->cfg.max_tokens) * H * 2, 1024);
  c->off_rowcnt = off;
  off = align_up(off + 64, 1024);
  c->off_keybox = off;
  off = align_up(off + 2 * W * static_cast<size_t>(c->cfg.max_seqs > 0 ? c->cfg.max_seqs : 1) * 8, 1024);
  c->off_tokens = off;
  off = align_up(off + 2 * static_cast<size_t>(c->cfg.max_seqs > 0 ? c->cfg.max_seqs : 1) * 8, 1024);
  c->symm_bytes = off;
  B2_CUDA(cudaMalloc(&c->symm, c->symm_bytes));
  {
    const int rc = init_symmetric_region(c);
    if (rc != B2_OK) return rc;
  }
  for (int r = 0; r < B2_MAX_WORLD; ++r) c->peer[r] = nullptr;
  c->peer[c->cfg.rank] = c->symm;
  c->peers_ready = (c->cfg.world == 1);

  // ---- rank-local scratch -----------------------------------------------------
  c->splitk_ws_bytes = static_cast<size_t>(c->num_sms) * 128 * 256 * sizeof(float);  // one 128 x 256 fp32 slot per CTA
  B2_CUDA(cudaMalloc(&c->splitk_ws, c->splitk_ws_bytes));
  B2_CUDA(cudaMemset(c->splitk_ws, 0, c->splitk_ws_bytes));  // accumulation slots start (and are left) at zero
  c->tile_counter_cap = 1 << 16;
  B2_CUDA(cudaMalloc(&c->tile_counters, static_cast<size_t>(c->tile_counter_cap) * 4 * sizeof(int)));
  B2_CUDA(cudaMemset(c->tile_counters, 0, static_cast<size_t>(c->tile_counter_cap) * 4 * sizeof(int)));
  B2_CUDA(cudaMalloc(&c->dstate, sizeof(B2DeviceState)));
  B2_CUDA(cudaMemset(c->dstate, 0, sizeof(B2DeviceState)));
  B2_CUDA(cudaHostAlloc(&c->status_host, sizeof(B2Status), cudaHostAllocMapped));
  memset(c->status_host, 0, sizeof(B2Status));
  c->status_host->rank = c->cfg.rank;
  B2_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0));
  if (c->cfg.max_seqs > 0) B2_CUDA(cudaMalloc(&c->gather_rows, static_cast<size_t>(c->cfg.max_seqs) * H * 2));
  if (c->cfg.max_seqs > 0) {
    B2_CUDA(cudaMalloc(&c->sample_keys, static_cast<size_t>(c->cfg.max_seqs) * 8));
    B2_CUDA(cudaMemset(c->sample_keys, 0, static_cast<size_t>(c->cfg.max_seqs) * 8));
  }
  B2_CUDA(cudaMalloc(&c->trace, static_cast<size_t>(c->num_sms) * 16 * sizeof(unsigned long long)));
  B2_CUDA(cudaMemset(c->trace, 0, static_cast<size_t>(c->num_sms) * 16 * sizeof(unsigned long long)));
  c->trace_on = false;
  B2_CUDA(cudaDeviceSynchronize());
  return B2_OK;
}

int b2_symm_export(b2_ctx* c, void* handle_out) {
  if (c == nullptr || handle_out == nullptr) return B2_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == B2_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  B2_CUDA(cudaIpcGetMemHandle(&h, c->symm));
  memcpy(handle_out, &h, sizeof(h));
  return B2_OK;
}

int b2_symm_import(b2_ctx* c, const void* handles) {
  if (c == nullptr || handles == nullptr) return B2_ERR_ARG;
  if (c->peers_ready) return B2_OK;
  for (int r = 0; r < c->cfg.world; ++r) {
    if (r == c->cfg.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const unsigned char*>(handles) + static_cast<size_t>(r) * B2_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    B2_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer[r] = static_cast<unsigned char*>(p);
  }
  c->peers_ready = true;
  return B2_OK;
}

int b2_ctx_destroy(b2_ctx* c) {
  if (c == nullptr) return B2_ERR_ARG;
  cudaSetDevice(c->cfg.device);
  cudaDeviceSynchronize();
  for (int r = 0; r < c->cfg.world; ++r)
    if (r != c->cfg.rank && c->peer[r] != nullptr) cudaIpcCloseMemHandle(c->peer[r]);
  cudaFree(c->symm);
  cudaFree(c->splitk_ws);
  cudaFree(c->tile_counters);
  cudaFree(c->dstate);
  cudaFree(c->trace);
  if (c->gather_rows) cudaFree(c->gather_rows);
  if (c->sample_keys) cudaFree(c->sample_keys);
  if (c->status_host) cudaFreeHost(c->status_host);
  cudaGetLastError();  // a failed free of a never-made allocation is not an error of the caller
  delete c;
  return B2_OK;
}

int b2_status(b2_ctx* c, int* code, int* detail) {
  if (c == nullptr) return B2_ERR_ARG;
  const volatile B2Status* s = c->status_host;
  if (code) *code = s->code;
  if (detail) *detail = s->detail;
  return B2_OK;
}

int b2_trace(b2_ctx* c, int enable, unsigned long long* host_out, int max_ctas) {
  if (c == nullptr) return B2_ERR_ARG;
  if (host_out != nullptr) {
    const int n = max_ctas < c->num_sms ? max_ctas : c->num_sms;
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaMemcpy(host_out, c->trace, static_cast<size_t>(n) * 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    B2_CUDA(cudaMemset(c->trace, 0, static_cast<size_t>(c->num_sms) * 16 * sizeof(unsigned long long)));
  }
  c->trace_on = enable != 0;
  return B2_OK;
}

int b2_ctx_reset(b2_ctx* c) {
  if (c == nullptr) return B2_ERR_ARG;
  B2_CUDA(cudaSetDevice(c->cfg.device));
  B2_CUDA(cudaDeviceSynchronize());
  const int rc = init_symmetric_region(c);
  if (rc != B2_OK) return rc;
  B2_CUDA(cudaMemset(c->splitk_ws, 0, c->splitk_ws_bytes));
  B2_CUDA(cudaMemset(c->tile_counters, 0, static_cast<size_t>(c->tile_counter_cap) * 4 * sizeof(int)));
  B2_CUDA(cudaMemset(c->dstate, 0, sizeof(B2DeviceState)));
  if (c->sample_keys) B2_CUDA(cudaMemset(c->sample_keys, 0, static_cast<size_t>(c->cfg.max_seqs) * 8));
  B2_CUDA(cudaDeviceSynchronize());
  c->status_host->code = 0;
  c->status_host->detail = 0;
  return B2_OK;
}

int b2_status_clear(b2_ctx* c) {
  if (c == nullptr) return B2_ERR_ARG;
  c->status_host->code = 0;
  c->status_host->detail = 0;
  return B2_OK;
}

}  // extern "C"
