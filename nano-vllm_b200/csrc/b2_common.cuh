// Shared device helpers: PTX wrappers for mbarrier / TMA / tcgen05 (sm_100a),
// bf16 packing, bounded waits, and the context layout.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200tp.h"

// ---------------------------------------------------------------------------
// wait codes written to the status word (detail field of b2_status)
// ---------------------------------------------------------------------------
enum : int {
  B2_WAIT_NONE = 0,
  B2_WAIT_SMEM_FULL = 1,    // MMA warp waiting for a TMA stage
  B2_WAIT_SMEM_EMPTY = 2,   // TMA warp waiting for a free stage
  B2_WAIT_TMEM_FULL = 3,    // epilogue waiting for an accumulator
  B2_WAIT_TMEM_EMPTY = 4,   // MMA warp waiting for a drained accumulator
  B2_WAIT_PARTIALS = 5,     // fused reduce waiting for partial rows (local or peer)
  B2_WAIT_EMBED = 6,        // embedding waiting for the owner rank's row
  B2_WAIT_LOGITS = 7,       // rank 0 waiting for peers' logits slices
  B2_WAIT_TOKENS = 8,       // a rank waiting for rank 0's sampled tokens
  B2_WAIT_ROWS = 9          // two-shot: waiting for the other owners' finished rows
};

// The bf16 bit pattern that marks "not written yet" in data-as-flag buffers:
// negative zero.  Producers never store it (they turn -0.0 into +0.0).
#define B2_SENTINEL16 0x8000u
#define B2_SENTINEL32 0x80008000u

// Device-resident state of one context (lives in ordinary device memory).
struct B2DeviceState {
  unsigned int rowpar_seq;     // number of fused row-parallel launches so far
  unsigned int rowpar_done;    // CTAs of the current launch that have finished
  unsigned int embed_seq;
  unsigned int embed_done;
  unsigned int lmhead_seq;
  unsigned int lmhead_done;
  unsigned int bcast_seq;
  unsigned int sample_seq;     // fused LM-head sampler calls so far (part of the noise counter, so graph replays draw afresh)
};

// Host-visible (mapped, pinned) status word.
struct B2Status {
  int code;
  int detail;
  int rank;
  int pad;
};

#define B2_MAX_WORLD 8

// ---------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------
namespace b2 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Has more than `limit_ns` passed since t0?  The 64-bit timer is not read in one piece on every part: a value read
// while its low half wraps can be off by 2^32 ns in either direction.  A limit counts as passed only if two
// successive readings both say so and neither lies before t0.
__device__ __forceinline__ bool time_limit_passed(uint64_t t0, uint64_t limit_ns) {
  const uint64_t a = globaltimer_ns();
  if (a < t0 || a - t0 <= limit_ns) return false;
  const uint64_t b = globaltimer_ns();
  return b >= a && b - t0 > limit_ns;
}

__device__ __forceinline__ void report_timeout(B2Status* st, int detail) {
  // the word is in mapped host memory; concurrent reporters write the same code
  if (st != nullptr) {
    volatile B2Status* v = st;
    v->detail = detail;
    v->code = B2_ERR_TIMEOUT;
    __threadfence_system();
  }
}

// ---- programmatic dependent launch -------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start
// while the kernel before it in the stream is still running.  Everything it
// does before pdl_wait() must be independent of earlier kernels (set-up,
// loads of weights); pdl_wait() returns once every earlier kernel has
// completed and its writes are visible.  Both are no-ops for a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- thread-block clusters / distributed shared memory --------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// every thread of every CTA of the cluster executes both; writes made before arrive are visible after wait
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// address of this CTA's shared-memory location `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float x, float y, float z, float w) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// ---- mbarrier --------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
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

// Bounded wait on an mbarrier phase.  Returns false when the CTA-wide abort
// flag is (or becomes) set: either this wait ran past `limit_ns` or another
// role of the CTA gave up first.  A legitimate wait inside the GEMM pipeline
// lasts microseconds; the limit only exists so that a bug cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3FF) == 0) {
      if (*abort_flag) return false;
      if (time_limit_passed(t0, limit_ns)) {
        *abort_flag = code;
        return false;
      }
    }
  }
}

// ---- TMA -------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// L2 eviction-priority policies for bulk tensor loads
constexpr uint64_t kEvictNormal = 0x1000000000000000ull;
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

// 2-D tiled load global -> this CTA's shared memory, completion on an mbarrier.
// x is the innermost (contiguous) coordinate and must keep the copy 16-byte
// aligned: x * 2 bytes is a multiple of 128 here (x is a multiple of 64).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// ---- tcgen05 / tensor memory -------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- the same for a CTA pair (cta_group::2): two CTAs of a cluster, ranks 2i and 2i+1, run one 256-row MMA.
// Every tcgen05 instruction of a kernel must name the same group, so a pair kernel uses only these forms.
// Allocation and release are issued by the same warp index in BOTH CTAs (each gets the address in its own slot).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Issued by one thread of the pair's even CTA.  Each CTA contributes the 128 rows of A and half of the rows of B
// that lie in its own shared memory at the descriptors' offsets; each CTA's tensor memory receives its 128 rows of D.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the mbarrier at this shared-memory offset in every CTA of `cta_mask`, once all MMAs issued so far
// by this thread have completed (a signal, not a data copy).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask) : "memory");
}
// 2-D tiled load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier that may live in
// the pair's other CTA (`bar_cluster` is a shared::cluster address, e.g. from map_to_cta).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// arrival on an mbarrier of another CTA of the cluster
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives the 32
// columns of TMEM lane (lane_base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory operand descriptor for a K-major bf16 tile whose rows are 128
// bytes (64 elements) apart, laid out by TMA with the 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart (stride byte offset), the leading byte
// offset is unused for swizzled K-major layouts (set to 16 bytes), descriptor
// version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset (>>4), bits [16,30)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset (>>4), bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                     // version, bits [46,48)
  d |= static_cast<uint64_t>(2) << 61;                     // layout type, bits [61,64)
  return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, bf16 A and
// B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int n) {
  return (1u << 4)                                  // D format: F32
         | (1u << 7)                                // A format: BF16
         | (1u << 10)                               // B format: BF16
         | (static_cast<uint32_t>(n >> 3) << 17)    // N / 8
         | (static_cast<uint32_t>(128 >> 4) << 24); // M / 16
}

// The same for a CTA pair: M = 256 (128 rows per CTA), N = n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

// ---- bf16 packing / data-as-flag helpers --------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// replace a -0.0 half (the sentinel) by +0.0 in a packed pair
__device__ __forceinline__ uint32_t scrub_sentinel(uint32_t w) {
  if ((w & 0xFFFFu) == B2_SENTINEL16) w &= 0xFFFF0000u;
  if ((w >> 16) == B2_SENTINEL16) w &= 0x0000FFFFu;
  return w;
}
__device__ __forceinline__ bool has_sentinel(uint32_t w) {
  return (w & 0xFFFFu) == B2_SENTINEL16 || (w >> 16) == B2_SENTINEL16;
}
__device__ __forceinline__ bool has_sentinel(const uint4& v) {
  return has_sentinel(v.x) || has_sentinel(v.y) || has_sentinel(v.z) || has_sentinel(v.w);
}
// 16-byte load that is never served from a stale L1 line (data another SM or
// another GPU writes while this kernel runs)
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

}  // namespace b2

// ---------------------------------------------------------------------------
// host-side context
// ---------------------------------------------------------------------------
struct b2_ctx {
  b2_config cfg;
  int num_sms;
  bool peers_ready;

  // symmetric region of this rank and the mapped addresses of every rank's
  // region (peer[rank] == symm)
  unsigned char* symm;
  size_t symm_bytes;
  unsigned char* peer[B2_MAX_WORLD];

  // offsets inside the symmetric region
  size_t off_rowpar;    // [2 parity][world][oneshot_tokens][hidden] bf16
  size_t off_embed;     // [2 parity][max_tokens][hidden] bf16
  size_t off_inbox2;    // two-shot: [2 parity][world][ceil(max_tokens/world)][hidden] bf16 partial rows for the rows this rank owns
  size_t off_logits;    // [max_seqs][vocab] bf16 (used on rank 0)
  size_t off_flags;     // [world] uint32 arrival flags for the logits gather
  size_t off_out;       // two-shot: [max_tokens][hidden] bf16 normed rows, written by their owner ranks
  size_t off_rowcnt;    // two-shot: [2 parity] uint32 rows received in off_out
  size_t off_keybox;    // fused sampler, used on rank 0: [2 parity][world][max_seqs] uint64 best (score, vocab id) of every rank
  size_t off_tokens;    // [2 parity][max_seqs] int64 token inbox, -1 = not written
  size_t off_inbox3;    // owner form: [2 parity][world][ceil(oneshot_tokens/world)][hidden] bf16 partial rows of the rows this rank owns
  size_t off_land;      // owner form: [2 parity][2 planes: normed, residual][oneshot_tokens][hidden] bf16 finished rows, written by their owners

  // which form of the fused row-parallel block b2_rowpar_fused launches (b2_ctx_set_option)
  int rowpar_form;         // B2_FORM_AUTO / ONESHOT / OWNER
  int owner_min_tokens;    // AUTO: the row-owner form serves owner_min_tokens .. owner_max_tokens tokens at world >= 2
  int owner_max_tokens;
  bool whole_tiles;        // fused row-parallel calls in the token-row layout: one whole tile per CTA when the tiles fit one wave
  int twoshot_min_tokens;  // b2_rowpar_form: from this many tokens on callers should use b2_rowpar_fused_twoshot

  // rank-local scratch
  float* splitk_ws;     // stream-K partial accumulators
  size_t splitk_ws_bytes;
  int* tile_counters;   // 4 per output tile, zero between launches
  int tile_counter_cap; // tiles
  B2DeviceState* dstate;
  B2Status* status_host;  // mapped pinned host memory
  B2Status* status_dev;   // device alias of status_host
  __nv_bfloat16* gather_rows;  // [max_seqs][hidden] staging for the LM head
  unsigned long long* sample_keys;  // [max_seqs] fused sampler: this rank's best key per row, zero between calls
  unsigned long long* trace;   // [num_sms][8][2] phase stamps of the last GEMM launch
  bool trace_on;
};

namespace b2 {
int set_cuda_error(cudaError_t e, const char* what);
int set_error(int code, const char* fmt, ...);  // formats the text b2_last_error() returns; returns code
void count_launch();
bool pdl_enabled();  // false when the environment has B2_PDL=0
int encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t ld_elems,
                   uint32_t box_inner, uint32_t box_rows);
}  // namespace b2

#define B2_CUDA(call)                                            \
  do {                                                           \
    cudaError_t e__ = (call);                                    \
    if (e__ != cudaSuccess) return b2::set_cuda_error(e__, #call); \
  } while (0)

// Launch with the programmatic-dependent-launch attribute (when enabled), so
// that consecutive kernels of this library overlap set-up with the previous
// kernel's tail.  Captured into CUDA graphs as a programmatic dependency.
template <typename... KArgs, typename... Args>
inline cudaError_t b2_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = b2::pdl_enabled() ? 2 : 1;
  b2::count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t b2_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = b2::pdl_enabled() ? 1 : 0;
  b2::count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
