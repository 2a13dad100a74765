// HBM-bound kernels of the path: paged-KV scatter, RMSNorm (plain and with the
// residual add), SiLU*mul, fused q/k-norm + RoPE + KV scatter, embedding
// lookup with owner-rank broadcast, greedy argmax.  All accesses are 16-byte
// vectors on the contiguous dimension.
#include <algorithm>

#include "b2_common.cuh"

namespace {

using b2::bf16_hi;
using b2::bf16_lo;
using b2::bf16_round;
using b2::pack_bf16;

__device__ __forceinline__ uint4 ldg_v4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void stg_v4(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// paged-KV scatter.  One thread moves one 16-byte vector of K and the matching
// vector of V of one token.  Threads of a warp cover consecutive vectors of a
// row, so every load and store is a full 32-byte-sector access.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) store_kvcache_kernel(const uint16_t* __restrict__ key, int64_t key_stride,
                                                            const uint16_t* __restrict__ value, int64_t value_stride,
                                                            uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                                                            const int32_t* __restrict__ slot_mapping, int n_tokens,
                                                            int vec_per_row) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int64_t total = static_cast<int64_t>(n_tokens) * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int token = static_cast<int>(i / vec_per_row);
    const int v = static_cast<int>(i - static_cast<int64_t>(token) * vec_per_row);
    const int slot = __ldg(slot_mapping + token);
    if (slot < 0) continue;  // -1 marks padded rows of a decode graph
    const uint4 kv = ldg_v4(key + token * key_stride + v * 8);
    const uint4 vv = ldg_v4(value + token * value_stride + v * 8);
    const int64_t dst = (static_cast<int64_t>(slot) * vec_per_row + v) * 8;
    stg_v4(k_cache + dst, kv);
    stg_v4(v_cache + dst, vv);
  }
}

// ---------------------------------------------------------------------------
// RMSNorm.  WARP_ROWS = true: one warp per row (dim <= 1024); otherwise one
// 256-thread block per row (dim <= 8192).  Each thread keeps its (up to 4)
// vectors in registers, so a row is read from HBM once.
// ---------------------------------------------------------------------------
template <bool ADD, bool WARP_ROWS>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* __restrict__ x, int64_t ldx,
                                                      const uint16_t* __restrict__ res, const uint16_t* __restrict__ w,
                                                      float eps, int rows, int dim, uint16_t* __restrict__ out, int64_t ldo,
                                                      uint16_t* __restrict__ res_out) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  constexpr int VPT = 4;
  const int lanes = WARP_ROWS ? 32 : 256;
  const int lane = WARP_ROWS ? (threadIdx.x & 31) : threadIdx.x;
  const int row = WARP_ROWS ? (blockIdx.x * 8 + (threadIdx.x >> 5)) : blockIdx.x;
  __shared__ float red[8];
  const int nvec = dim >> 3;
  const bool active = row < rows;
  float vals[VPT][8];
  float ss = 0.f;
  if (active) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = lane + j * lanes;
      if (v < nvec) {
        unpack8(ldg_v4(x + row * ldx + v * 8), vals[j]);
        if (ADD) {
          float r[8];
          unpack8(ldg_v4(res + static_cast<int64_t>(row) * dim + v * 8), r);
#pragma unroll
          for (int e = 0; e < 8; ++e) vals[j][e] += r[e];
          stg_v4(res_out + static_cast<int64_t>(row) * dim + v * 8, pack8(vals[j]));
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += vals[j][e] * vals[j][e];
      }
    }
  }
  ss = warp_sum(ss);
  if (!WARP_ROWS) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += red[i];
  }
  if (!active) return;
  const float rstd = rsqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = lane + j * lanes;
    if (v < nvec) {
      float wv[8], o[8];
      unpack8(ldg_v4(w + v * 8), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = bf16_round(vals[j][e] * rstd) * wv[e];
      stg_v4(out + row * ldo + v * 8, pack8(o));
    }
  }
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint16_t* __restrict__ x, int64_t ldx, int M, int I,
                                                       uint16_t* __restrict__ out) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int vpr = I >> 3;
  const int64_t total = static_cast<int64_t>(M) * vpr;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / vpr);
    const int v = static_cast<int>(i - static_cast<int64_t>(m) * vpr);
    float g[8], u[8], o[8];
    unpack8(ldg_v4(x + m * ldx + v * 8), g);
    unpack8(ldg_v4(x + m * ldx + I + v * 8), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = bf16_round(g[e] / (1.0f + expf(-g[e]))) * u[e];
    stg_v4(out + static_cast<int64_t>(m) * I + v * 8, pack8(o));
  }
}

// ---------------------------------------------------------------------------
// q/k head RMSNorm + neox RoPE (in place) + scatter of K and V into the paged
// cache.  One warp per (token, head).  HALF = head_dim / 2; lane l owns the
// element pairs (2l, 2l+1) of both halves (HALF = 64) or element l of both
// halves (HALF = 32).
// ---------------------------------------------------------------------------
template <int HALF>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(uint16_t* __restrict__ qkv, int64_t ld, int M, int nq, int nkv,
                                                                 const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                                                                 float eps, const int64_t* __restrict__ positions,
                                                                 const float* __restrict__ cos_sin, uint16_t* __restrict__ k_cache,
                                                                 uint16_t* __restrict__ v_cache, const int32_t* __restrict__ slots) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  constexpr int HD = 2 * HALF;
  constexpr int EPL = HALF / 32;  // elements per lane per half: 2 or 1
  const int heads = nq + 2 * nkv;
  const int64_t gw = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<int64_t>(M) * heads) return;
  const int token = static_cast<int>(gw / heads);
  const int head = static_cast<int>(gw - static_cast<int64_t>(token) * heads);
  uint16_t* p = qkv + token * ld + static_cast<int64_t>(head) * HD;
  const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
  const int slot = (k_cache != nullptr && !is_q) ? __ldg(slots + token) : -1;
  const int kvh = is_k ? head - nq : head - nq - nkv;
  const int64_t cache_off = (static_cast<int64_t>(slot) * nkv + kvh) * HD;

  if (!is_q && !is_k) {  // V head: copy to the cache only
    if (slot >= 0) {
      if (EPL == 2) {
        const uint2 v = *reinterpret_cast<const uint2*>(p + lane * 4);
        *reinterpret_cast<uint2*>(v_cache + cache_off + lane * 4) = v;
      } else {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(p + lane * 2);
        *reinterpret_cast<uint32_t*>(v_cache + cache_off + lane * 2) = v;
      }
    }
    return;
  }

  float x1[EPL], x2[EPL];
  if (EPL == 2) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(p + lane * 2);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(p + HALF + lane * 2);
    x1[0] = bf16_lo(a); x1[EPL - 1] = bf16_hi(a);
    x2[0] = bf16_lo(b); x2[EPL - 1] = bf16_hi(b);
  } else {
    x1[0] = __uint_as_float(static_cast<uint32_t>(p[lane]) << 16);
    x2[0] = __uint_as_float(static_cast<uint32_t>(p[HALF + lane]) << 16);
  }
  const uint16_t* nw = is_q ? qw : kw;
  if (nw != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / static_cast<float>(HD) + eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float w1 = __uint_as_float(static_cast<uint32_t>(nw[lane * EPL + e]) << 16);
      const float w2 = __uint_as_float(static_cast<uint32_t>(nw[HALF + lane * EPL + e]) << 16);
      x1[e] = bf16_round(bf16_round(x1[e] * rstd) * w1);
      x2[e] = bf16_round(bf16_round(x2[e] * rstd) * w2);
    }
  }
  const float* cs = cos_sin + positions[token] * HD;
  float y1[EPL], y2[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const float c = __ldg(cs + lane * EPL + e), s = __ldg(cs + HALF + lane * EPL + e);
    // separate roundings of the products, as the eager reference computes them
    y1[e] = __fsub_rn(__fmul_rn(x1[e], c), __fmul_rn(x2[e], s));
    y2[e] = __fadd_rn(__fmul_rn(x2[e], c), __fmul_rn(x1[e], s));
  }
  if (EPL == 2) {
    const uint32_t a = pack_bf16(y1[0], y1[EPL - 1]), b = pack_bf16(y2[0], y2[EPL - 1]);
    *reinterpret_cast<uint32_t*>(p + lane * 2) = a;
    *reinterpret_cast<uint32_t*>(p + HALF + lane * 2) = b;
    if (is_k && slot >= 0) {
      *reinterpret_cast<uint32_t*>(k_cache + cache_off + lane * 2) = a;
      *reinterpret_cast<uint32_t*>(k_cache + cache_off + HALF + lane * 2) = b;
    }
  } else {
    const uint16_t a = static_cast<uint16_t>(pack_bf16(y1[0], 0.f) & 0xFFFF), b = static_cast<uint16_t>(pack_bf16(y2[0], 0.f) & 0xFFFF);
    p[lane] = a;
    p[HALF + lane] = b;
    if (is_k && slot >= 0) {
      k_cache[cache_off + lane] = a;
      k_cache[cache_off + HALF + lane] = b;
    }
  }
}

// ---------------------------------------------------------------------------
// Embedding.  world == 1: plain row gather.  world > 1: the rank that owns a
// token id stores the row into every peer's inbox (data-as-flag: the inbox
// holds the sentinel until the row lands) and into its own output; the other
// ranks poll their inbox, copy the row out and put the sentinel back.  Two
// inboxes alternate by launch parity so that a rank that runs ahead writes
// the next launch's rows somewhere else.
// ---------------------------------------------------------------------------
struct EmbedArgs {
  const int64_t* ids;
  const uint16_t* W;
  int64_t vocab_start, vocab_end;
  int M, H;
  uint16_t* out;
  int world, rank;
  unsigned char* peer_inbox[B2_MAX_WORLD];  // base of each rank's embed inbox (both parities)
  size_t parity_stride;                     // bytes between the two inboxes
  B2DeviceState* dstate;
  B2Status* status;
  uint64_t timeout_ns;
};

__global__ void __launch_bounds__(256) embed_kernel(const EmbedArgs a) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int vpr = a.H >> 3;
  const int64_t total = static_cast<int64_t>(a.M) * vpr;
  const int64_t first = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (a.world == 1) {
    // four rows' vectors in flight per thread: the id load in front of every row read is a dependent load, so one
    // item at a time leaves the memory system a quarter full
    constexpr int U = 4;
    const int64_t span = a.vocab_end - a.vocab_start;
    for (int64_t i0 = first; i0 < total; i0 += step * U) {
      int64_t off[U];
      uint4 val[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + u * step;
        off[u] = -1;
        if (i < total) {
          const int m = static_cast<int>(i / vpr);
          const int v = static_cast<int>(i - static_cast<int64_t>(m) * vpr);
          int64_t row = a.ids[m] - a.vocab_start;
          if (row < 0 || row >= span) row = 0;  // the reference would fault; stay in bounds
          off[u] = static_cast<int64_t>(m) * a.H + v * 8;
          val[u] = ldg_v4(a.W + row * a.H + v * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (off[u] >= 0) stg_v4(a.out + off[u], val[u]);
    }
    return;
  }
  const unsigned int parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->embed_seq) & 1u;
  // pass 1: rows this rank owns go to every peer's inbox and to the local
  // output.  Nothing here waits, so no rank can block another's pushes.
  for (int64_t i = first; i < total; i += step) {
    const int m = static_cast<int>(i / vpr);
    const int v = static_cast<int>(i - static_cast<int64_t>(m) * vpr);
    const int64_t id = a.ids[m];
    if (id < a.vocab_start || id >= a.vocab_end) continue;
    const size_t inbox_off = parity * a.parity_stride + (static_cast<size_t>(m) * a.H + v * 8) * 2;
    uint4 val = ldg_v4(a.W + (id - a.vocab_start) * a.H + v * 8);
    stg_v4(a.out + static_cast<int64_t>(m) * a.H + v * 8, val);
    val.x = b2::scrub_sentinel(val.x); val.y = b2::scrub_sentinel(val.y);
    val.z = b2::scrub_sentinel(val.z); val.w = b2::scrub_sentinel(val.w);
    for (int r = 0; r < a.world; ++r)
      if (r != a.rank) stg_v4(a.peer_inbox[r] + inbox_off, val);
  }
  // pass 2: rows owned elsewhere arrive in the local inbox
  for (int64_t i = first; i < total; i += step) {
    const int m = static_cast<int>(i / vpr);
    const int v = static_cast<int>(i - static_cast<int64_t>(m) * vpr);
    const int64_t id = a.ids[m];
    if (id >= a.vocab_start && id < a.vocab_end) continue;
    unsigned char* src = a.peer_inbox[a.rank] + parity * a.parity_stride + (static_cast<size_t>(m) * a.H + v * 8) * 2;
    uint4 val = b2::ld_volatile_v4(src);
    if (b2::has_sentinel(val)) {
      const uint64_t t0 = b2::globaltimer_ns();
      for (uint32_t it = 1;; ++it) {
        val = b2::ld_volatile_v4(src);
        if (!b2::has_sentinel(val)) break;
        if ((it & 0xFF) == 0 && b2::time_limit_passed(t0, a.timeout_ns)) {
          b2::report_timeout(a.status, B2_WAIT_EMBED);
          break;
        }
      }
    }
    stg_v4(a.out + static_cast<int64_t>(m) * a.H + v * 8, val);
    stg_v4(src, make_uint4(B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32));
  }
  // the last block to finish advances the launch parity for the next call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&a.dstate->embed_done, 1u);
    if (prev == gridDim.x - 1) {
      a.dstate->embed_done = 0;
      a.dstate->embed_seq += 1;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------
// argmax over each row (first index wins ties).  A row is split over several blocks; each block folds its
// columns into one 64-bit key (value bits made order-preserving in the high word, ~index in the low word) and
// atomicMax-es it into the row's output word; a second tiny kernel turns the winning key back into the index.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone map float -> uint
  return (static_cast<unsigned long long>(b) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(idx));
}

__global__ void __launch_bounds__(256) argmax_partial_kernel(const uint16_t* __restrict__ logits, int64_t ld, int V, int cols_per_block,
                                                             unsigned long long* __restrict__ keys) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const uint16_t* row = logits + blockIdx.x * ld;
  const int c0 = blockIdx.y * cols_per_block, c1 = min(V, c0 + cols_per_block);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int v0 = c0 >> 3, v1 = c1 >> 3;  // cols_per_block is a multiple of 8
  for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    float f[8];
    unpack8(ldg_v4(row + v * 8), f);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f[e] > best) { best = f[e]; best_i = v * 8 + e; }
  }
  for (int i = max(c0, v1 * 8) + threadIdx.x; i < c1; i += blockDim.x) {
    const float f = __uint_as_float(static_cast<uint32_t>(row[i]) << 16);
    if (f > best || (f == best && i < best_i)) { best = f; best_i = i; }
  }
  unsigned long long key = best_i == 0x7fffffff ? 0ull : argmax_key(best, best_i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  __shared__ unsigned long long sk[8];
  if ((threadIdx.x & 31) == 0) sk[threadIdx.x >> 5] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) key = sk[i] > key ? sk[i] : key;
    atomicMax(keys + blockIdx.x, key);
  }
}

__global__ void argmax_finish_kernel(int64_t* __restrict__ out, int B) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B) {
    const unsigned long long key = static_cast<unsigned long long>(out[i]);
    out[i] = key == 0ull ? 0 : static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(key & 0xFFFFFFFFull));
  }
}

// ---------------------------------------------------------------------------
// Rank 0's int64 values to every rank.  The inbox holds -1 until a value lands;
// the reader copies it out and puts -1 back.  Two inboxes alternate by call.
// One block; n <= max_seqs.
// ---------------------------------------------------------------------------
struct BcastArgs {
  int64_t* buf;
  int n, world, rank;
  unsigned char* inbox[B2_MAX_WORLD];
  size_t parity_stride;
  B2DeviceState* dstate;
  B2Status* status;
  uint64_t timeout_ns;
};

__global__ void __launch_bounds__(256) broadcast_tokens_kernel(const BcastArgs a) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const unsigned int parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->bcast_seq) & 1u;
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
    if (a.rank == 0) {
      const long long v = a.buf[i];
      for (int r = 1; r < a.world; ++r)
        *reinterpret_cast<volatile long long*>(a.inbox[r] + parity * a.parity_stride + i * 8) = v;
    } else {
      volatile long long* src = reinterpret_cast<volatile long long*>(a.inbox[a.rank] + parity * a.parity_stride + i * 8);
      long long v = *src;
      if (v < 0) {
        const uint64_t t0 = b2::globaltimer_ns();
        for (uint32_t it = 1; (v = *src) < 0; ++it) {
          if ((it & 0xFF) == 0 && b2::time_limit_passed(t0, a.timeout_ns)) {
            b2::report_timeout(a.status, B2_WAIT_TOKENS);
            v = 0;
            break;
          }
        }
      }
      a.buf[i] = v;
      *src = -1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    a.dstate->bcast_seq += 1;
    __threadfence();
  }
}

// A row whose next position has no block in its table (past the table's width, a -1 entry, or a slot beyond the
// cache) is frozen: it stores nothing (slot -1) and its position and context length stay, so that a replay past
// a sequence's capacity can never send the KV scatter outside the cache.
__global__ void advance_decode_kernel(const int64_t* __restrict__ tokens, int64_t* __restrict__ input_ids,
                                      int64_t* __restrict__ positions, int32_t* __restrict__ context_lens,
                                      int32_t* __restrict__ slot_mapping, const int32_t* __restrict__ block_tables,
                                      int64_t bt_stride, int bt_width, int block_size, int64_t num_slots, int n) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  input_ids[i] = tokens[i];
  const int64_t p = positions[i] + 1;
  const int64_t b = p / block_size;
  int32_t blk = -1;
  if (p >= 0 && b < bt_width && slot_mapping[i] >= 0) blk = block_tables[i * bt_stride + b];
  const int64_t slot = static_cast<int64_t>(blk) * block_size + (p % block_size);
  if (blk < 0 || slot >= num_slots) {
    slot_mapping[i] = -1;
    return;
  }
  positions[i] = p;
  context_lens[i] += 1;
  slot_mapping[i] = static_cast<int32_t>(slot);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
int grid_for(int64_t work_items, int threads, int cap) {
  int64_t g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace

extern "C" {

int b2_store_kvcache(const void* key, int64_t key_stride, const void* value, int64_t value_stride, void* k_cache,
                     void* v_cache, const int32_t* slot_mapping, int n_tokens, int D, void* stream) {
  if (n_tokens < 0 || D <= 0 || D % 8 != 0) return B2_ERR_ARG;
  if (n_tokens == 0) return B2_OK;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping) return B2_ERR_ARG;
  if (!aligned16(key) || !aligned16(value) || !aligned16(k_cache) || !aligned16(v_cache)) return B2_ERR_ARG;
  if (key_stride % 8 != 0 || value_stride % 8 != 0 || key_stride < D || value_stride < D) return B2_ERR_ARG;
  const int vpr = D / 8;
  const int grid = grid_for(static_cast<int64_t>(n_tokens) * vpr, 256, 148 * 16);
  B2_CUDA(b2_launch(store_kvcache_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(key), key_stride, static_cast<const uint16_t*>(value), value_stride,
                    static_cast<uint16_t*>(k_cache), static_cast<uint16_t*>(v_cache), slot_mapping, n_tokens, vpr));
  return B2_OK;
}

static int launch_rmsnorm(bool add, const void* x, int64_t ldx, const void* res, const void* w, float eps, int rows, int dim,
                          void* out, int64_t ldo, void* res_out, void* stream) {
  if (rows < 0 || dim <= 0 || dim % 8 != 0 || dim > 8192) return B2_ERR_ARG;
  if (rows == 0) return B2_OK;
  if (!x || !w || !out || (add && (!res || !res_out))) return B2_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(out) || ldx % 8 != 0 || ldo % 8 != 0) return B2_ERR_ARG;
  if (add && (!aligned16(res) || !aligned16(res_out))) return B2_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint16_t* xx = static_cast<const uint16_t*>(x);
  const uint16_t* rr = static_cast<const uint16_t*>(res);
  const uint16_t* ww = static_cast<const uint16_t*>(w);
  uint16_t* oo = static_cast<uint16_t*>(out);
  uint16_t* ro = static_cast<uint16_t*>(res_out);
  if (dim <= 1024) {
    const int grid = (rows + 7) / 8;
    if (add) B2_CUDA(b2_launch(rmsnorm_kernel<true, true>, dim3(grid), dim3(256), 0, s, xx, ldx, rr, ww, eps, rows, dim, oo, ldo, ro));
    else B2_CUDA(b2_launch(rmsnorm_kernel<false, true>, dim3(grid), dim3(256), 0, s, xx, ldx, rr, ww, eps, rows, dim, oo, ldo, ro));
  } else {
    if (add) B2_CUDA(b2_launch(rmsnorm_kernel<true, false>, dim3(rows), dim3(256), 0, s, xx, ldx, rr, ww, eps, rows, dim, oo, ldo, ro));
    else B2_CUDA(b2_launch(rmsnorm_kernel<false, false>, dim3(rows), dim3(256), 0, s, xx, ldx, rr, ww, eps, rows, dim, oo, ldo, ro));
  }
  return B2_OK;
}

int b2_rmsnorm(const void* x, int64_t ldx, const void* w, float eps, int rows, int dim, void* out, int64_t ldo, void* stream) {
  return launch_rmsnorm(false, x, ldx, nullptr, w, eps, rows, dim, out, ldo, nullptr, stream);
}

int b2_add_rmsnorm(const void* x, const void* res, const void* w, float eps, int rows, int dim, void* out, void* res_out,
                   void* stream) {
  return launch_rmsnorm(true, x, dim, res, w, eps, rows, dim, out, dim, res_out, stream);
}

int b2_silu_and_mul(const void* x, int64_t ldx, int M, int I, void* out, void* stream) {
  if (M < 0 || I <= 0 || I % 8 != 0 || ldx % 8 != 0 || ldx < 2 * static_cast<int64_t>(I)) return B2_ERR_ARG;
  if (M == 0) return B2_OK;
  if (!x || !out || !aligned16(x) || !aligned16(out)) return B2_ERR_ARG;
  const int grid = grid_for(static_cast<int64_t>(M) * (I / 8), 256, 148 * 16);
  B2_CUDA(b2_launch(silu_mul_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(x), ldx, M, I,
                    static_cast<uint16_t*>(out)));
  return B2_OK;
}

int b2_qk_norm_rope_store(void* qkv, int64_t ld_qkv, int M, int nq, int nkv, int head_dim, const void* q_norm_w,
                          const void* k_norm_w, float eps, const int64_t* positions, const float* cos_sin, void* k_cache,
                          void* v_cache, const int32_t* slot_mapping, void* stream) {
  if (M < 0 || nq <= 0 || nkv <= 0 || (head_dim != 128 && head_dim != 64)) return B2_ERR_ARG;
  if (M == 0) return B2_OK;
  if (!qkv || !positions || !cos_sin || ld_qkv < static_cast<int64_t>(nq + 2 * nkv) * head_dim || ld_qkv % 8 != 0) return B2_ERR_ARG;
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return B2_ERR_ARG;
  if (k_cache != nullptr && (!v_cache || !slot_mapping)) return B2_ERR_ARG;
  const int64_t warps = static_cast<int64_t>(M) * (nq + 2 * nkv);
  const int grid = static_cast<int>((warps + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint16_t* qp = static_cast<uint16_t*>(qkv);
  const uint16_t* qw = static_cast<const uint16_t*>(q_norm_w);
  const uint16_t* kw = static_cast<const uint16_t*>(k_norm_w);
  uint16_t* kc = static_cast<uint16_t*>(k_cache);
  uint16_t* vc = static_cast<uint16_t*>(v_cache);
  if (head_dim == 128)
    B2_CUDA(b2_launch(qk_norm_rope_store_kernel<64>, dim3(grid), dim3(256), 0, s, qp, ld_qkv, M, nq, nkv, qw, kw, eps, positions, cos_sin, kc, vc, slot_mapping));
  else
    B2_CUDA(b2_launch(qk_norm_rope_store_kernel<32>, dim3(grid), dim3(256), 0, s, qp, ld_qkv, M, nq, nkv, qw, kw, eps, positions, cos_sin, kc, vc, slot_mapping));
  return B2_OK;
}

int b2_embed(b2_ctx* ctx, const int64_t* ids, const void* W, int64_t vocab_start, int64_t vocab_end, int M, int H, void* out,
             void* stream) {
  if (M < 0 || H <= 0 || H % 8 != 0 || vocab_end <= vocab_start) return B2_ERR_ARG;
  if (M == 0) return B2_OK;
  if (!ids || !W || !out || !aligned16(W) || !aligned16(out)) return B2_ERR_ARG;
  EmbedArgs a{};
  a.ids = ids; a.W = static_cast<const uint16_t*>(W);
  a.vocab_start = vocab_start; a.vocab_end = vocab_end;
  a.M = M; a.H = H; a.out = static_cast<uint16_t*>(out);
  a.world = ctx ? ctx->cfg.world : 1;
  a.rank = ctx ? ctx->cfg.rank : 0;
  if (a.world > 1) {
    if (!ctx->peers_ready) return B2_ERR_STATE;
    if (M > ctx->cfg.max_tokens || H > ctx->cfg.hidden) return B2_ERR_SHAPE;
    for (int r = 0; r < a.world; ++r) a.peer_inbox[r] = ctx->peer[r] + ctx->off_embed;
    a.parity_stride = static_cast<size_t>(ctx->cfg.max_tokens) * ctx->cfg.hidden * 2;
    a.dstate = ctx->dstate;
    a.status = ctx->status_dev;
    a.timeout_ns = static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull;
  }
  const int cap = ctx ? ctx->num_sms * 4 : 148 * 4;
  const int grid = grid_for(static_cast<int64_t>(M) * (H / 8), 256, cap);
  B2_CUDA(b2_launch(embed_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), a));
  return B2_OK;
}

int b2_broadcast_tokens(b2_ctx* ctx, int64_t* buf, int n, void* stream) {
  if (ctx == nullptr || n < 0) return B2_ERR_ARG;
  if (ctx->cfg.world == 1 || n == 0) return B2_OK;
  if (buf == nullptr) return B2_ERR_ARG;
  if (!ctx->peers_ready) return B2_ERR_STATE;
  if (n > ctx->cfg.max_seqs) return B2_ERR_SHAPE;
  BcastArgs a{};
  a.buf = buf; a.n = n; a.world = ctx->cfg.world; a.rank = ctx->cfg.rank;
  for (int r = 0; r < a.world; ++r) a.inbox[r] = ctx->peer[r] + ctx->off_tokens;
  a.parity_stride = static_cast<size_t>(ctx->cfg.max_seqs) * 8;
  a.dstate = ctx->dstate;
  a.status = ctx->status_dev;
  a.timeout_ns = static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull;
  B2_CUDA(b2_launch(broadcast_tokens_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), a));
  return B2_OK;
}

int b2_advance_decode(const int64_t* tokens, int64_t* input_ids, int64_t* positions, int32_t* context_lens,
                      int32_t* slot_mapping, const int32_t* block_tables, int64_t bt_stride, int bt_width, int block_size,
                      int64_t num_slots, int n, void* stream) {
  if (n < 0 || block_size <= 0 || bt_width <= 0 || bt_stride < bt_width || num_slots <= 0) return B2_ERR_ARG;
  if (n == 0) return B2_OK;
  if (!tokens || !input_ids || !positions || !context_lens || !slot_mapping || !block_tables) return B2_ERR_ARG;
  B2_CUDA(b2_launch(advance_decode_kernel, dim3((n + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), tokens, input_ids, positions,
                    context_lens, slot_mapping, block_tables, bt_stride, bt_width, block_size, num_slots, n));
  return B2_OK;
}

int b2_argmax(const void* logits, int64_t ld, int B, int V, int64_t* out, void* stream) {
  if (B < 0 || V <= 0 || ld % 8 != 0 || ld < V) return B2_ERR_ARG;
  if (B == 0) return B2_OK;
  if (!logits || !out || !aligned16(logits)) return B2_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // enough blocks per row to fill the GPU, at least 4096 columns each
  int parts = std::max(1, std::min(32, 592 / std::max(1, B)));
  int cols = ((V + parts - 1) / parts + 7) / 8 * 8;
  if (cols < 4096) cols = 4096;
  parts = (V + cols - 1) / cols;
  B2_CUDA(cudaMemsetAsync(out, 0, static_cast<size_t>(B) * sizeof(int64_t), s));  // key 0 loses against every real key
  B2_CUDA(b2_launch(argmax_partial_kernel, dim3(B, parts), dim3(256), 0, s, static_cast<const uint16_t*>(logits), ld, V, cols,
                    reinterpret_cast<unsigned long long*>(out)));
  B2_CUDA(b2_launch(argmax_finish_kernel, dim3((B + 127) / 128), dim3(128), 0, s, out, B));
  return B2_OK;
}

}  // extern "C"
