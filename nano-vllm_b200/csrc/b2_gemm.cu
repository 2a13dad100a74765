// bf16 GEMMs for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with fp32
// accumulators in tensor memory, warp-specialised (1 TMA thread, 1 MMA thread,
// 4 epilogue warps).  Two kernels share the operand convention and epilogues:
//
//   gemm_kernel          persistent over a stream-K partition of the work (any size)
//   gemm_cluster_kernel  one thread-block cluster per output tile, K split over the
//                        cluster, parts combined through distributed shared memory
//                        (decode sizes: at most 64 tokens and one wave of tiles)
//
// D[p, q] = sum_k P[p, k] * Q[q, k]; both operands are K-major (row-major with
// K contiguous).  P tiles have 128 rows (the MMA M dimension = 128 TMEM
// lanes), Q tiles have BN rows (the MMA N dimension = BN TMEM columns).
//   SWAP = false ("token-row" layout): P = activations [tokens, K], Q = weights
//   SWAP = true ("feature-lane" layout): P = weights, Q = activations (few tokens:
//                 the 128-row side is filled by weight rows, so no tensor-core work
//                 is wasted and every SM streams a distinct slab of the weights)
//
// Stream-K: work unit = one 64-wide K block of one output tile.  The units are
// dealt in contiguous ranges to the CTAs; a tile whose K range is shared by
// several CTAs is combined in an fp32 accumulation slot in L2 (vector red.add):
// the CTA that arrives last at the tile's counter reads the sum, re-zeroes the
// slot and writes the output.  Nobody waits for anybody.  Up to 4 accumulators
// in tensor memory let a tile's epilogue overlap the next tile's MMAs.
//
// Epilogues:
//   EPI_STORE  C = D (+ bias); optionally SiLU(gate) * up on interleaved
//              (gate, up) feature pairs; in the cluster kernel optionally the
//              per-head work of the qkv projection (q/k RMSNorm, RoPE, KV scatter).
//   EPI_PUSH   the fused row-parallel path, one-shot.  The epilogue rounds the
//              tile to bf16 and stores it into the inbox of every rank (its own
//              and, over NVLink, its peers'); then every CTA turns to whole rows
//              of the inbox: it sums the partials of all ranks, adds the residual,
//              applies RMSNorm and writes the results.  The inbox is data-as-flag:
//              a slot holds the sentinel until the value lands, and the reader puts
//              the sentinel back after consuming it.
//   EPI_PUSH2  the two-shot form for many tokens.  Token rows are dealt to the
//              ranks in 16-row blocks, round-robin.  The epilogue stores each
//              partial row only into the inbox of the rank that owns it; the owner
//              sums the partials of its rows, adds the residual, normalises, and
//              stores the finished row into every rank's output buffer (symmetric
//              memory), then adds the number of rows it finished to each peer's
//              arrival counter.  A launch ends when its rank has received all rows
//              it does not own.  NVLink carries 2 (tp-1)/tp M N 2 bytes per rank,
//              the minimum for an all-reduce.
//   EPI_PUSH3  the row-owner form for few tokens (decode) at tensor-parallel size >= 4, where pushing a copy of
//              the partial to every rank costs more than a second NVLink hop.  Token row t belongs to rank
//              t mod world.  The epilogue stores each partial row only into its owner's inbox; the owner sums
//              the partials, adds the residual, normalises, and stores the finished row AND the new residual
//              row into every rank's landing buffer (symmetric memory, data-as-flag like the inbox); every
//              rank then copies the rows that have landed into the caller's tensors and puts the sentinel
//              back.  No fence, flag or counter is on the critical path: two NVLink store latencies per call
//              and 2 (tp-1)/tp M N 2 (+ the residual's share) bytes per rank.  Same outputs as EPI_PUSH.
//   EPI_SAMPLE the LM head fused with the sampler: no logits are stored.  Every
//              (token, vocab entry) score - the bf16-rounded logit, divided by the
//              row's temperature plus Gumbel noise from a counter-based generator,
//              or the logit alone for greedy decoding - is packed with its vocab id
//              into a 64-bit key whose unsigned order is (score, lowest id first);
//              the kernel keeps the largest key per token row.
//
// Every kernel is launched with the programmatic-dependent-launch attribute:
// set-up and the first ring of weight tiles are issued before
// griddepcontrol.wait, i.e. while the previous kernel of the stream is ending.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "b2_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int MAX_ROW_VECS = 6;  // 16-byte vectors of one row per thread in the reduce phase
constexpr uint64_t PIPE_LIMIT_NS = 1000000000ull;  // no wait inside the GEMM pipeline lasts anywhere near this

enum { EPI_STORE = 0, EPI_PUSH = 1, EPI_PUSH2 = 2, EPI_SAMPLE = 3, EPI_PUSH3 = 4 };
__host__ __device__ constexpr bool is_push(int epi) { return epi == EPI_PUSH || epi == EPI_PUSH2 || epi == EPI_PUSH3; }  // epilogues of the fused row-parallel call

struct GemmArgs {
  int tilesP, tilesQ, kblocks;
  int gemm_ctas;  // the first gemm_ctas CTAs of the grid share the GEMM units
  int round_robin;  // 1: whole tiles dealt round-robin instead of a stream-K range
  int M, N;       // tokens, features of the output
  // EPI_STORE
  uint16_t* C;
  int64_t ldc;
  const uint16_t* bias;
  // qkv projection fused with q/k head norm + RoPE + KV scatter (cluster kernel only; one 128-wide head per tile)
  int qkv_fused, nq, nkv;
  const int64_t* positions;
  const float* cos_sin;
  const uint16_t* q_norm_w;
  const uint16_t* k_norm_w;
  float qk_eps;
  uint16_t* k_cache;
  uint16_t* v_cache;
  const int32_t* slots;
  int silu_pairs;  // 1: features come in (gate, up) pairs; store silu(gate) * up, one value per pair, at column feature / 2
  // stream-K combine
  float* ws;
  int* counters;
  B2Status* status;
  // EPI_PUSH
  unsigned char* inbox[B2_MAX_WORLD];
  size_t parity_stride, slot_stride;
  int world, rank;
  const uint16_t* residual_in;
  const uint16_t* norm_w;
  float eps;
  uint16_t* normed_out;
  uint16_t* residual_out;
  B2DeviceState* dstate;
  uint64_t timeout_ns;
  // EPI_PUSH2 (inbox / parity_stride / slot_stride then describe the row-owner inbox)
  size_t out_off, rowcnt_off;  // from inbox[r]: that rank's [max_tokens][hidden] output buffer and its [2] rows-received counters
  int rows_per_rank;
  // EPI_PUSH3 (inbox / parity_stride / slot_stride describe the owners' inbox): from inbox[r], that rank's landing buffer
  // [2 parity][2 planes: normed, residual][tokens][N] bf16
  size_t land_off, land_parity_stride, land_plane_stride;
  unsigned long long* trace;  // optional [CTA][8][2] (SM clock, global ns) phase stamps; null = off
  // EPI_SAMPLE (LM head fused with the sampler; feature-lane layout only, features = vocabulary entries)
  unsigned long long* sample_keys;  // [M] best (score, vocab id) per token row, zero between calls
  const float* temperatures;        // [M], or null = greedy
  unsigned long long seed;
  int vocab_offset;                 // vocabulary id of feature 0 (rank * vocab / world)
};

template <int BN>
struct Cfg {
  static constexpr uint32_t P_BYTES = BM * BK * 2;
  static constexpr uint32_t Q_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = P_BYTES + Q_BYTES;
  static constexpr int STAGES = (196608 / STAGE_BYTES) > 8 ? 8 : (196608 / STAGE_BYTES);
  static constexpr int ACC = BN <= 128 ? 4 : 2;  // accumulators in tensor memory (512 columns in all)
  static constexpr uint32_t TMEM_COLS = ACC * BN;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t SMEM_BYTES_ROWS = SMEM_BYTES + 4 * 8192 /*epilogue staging of the token-row layout*/;
};

struct Partition {
  int base, rem;
  __host__ __device__ int u0(int c) const { return c * base + (c < rem ? c : rem); }
  __host__ __device__ int cta_of(int u) const {
    const int big = rem * (base + 1);
    return u < big ? u / (base + 1) : rem + (u - big) / base;
  }
};

struct Seg {
  int tile, kb0, kb1;
};

// The K blocks a CTA works through, by local index i = 0 .. n_units-1.
//   stream-K   : a contiguous range of the global unit order (tile-major), cut anywhere, also inside a tile
//   round-robin: whole tiles cta, cta + G, cta + 2G, ... (many-tile problems: the CTAs sweep the token
//                rows together, front to back, so finished rows become available steadily)
struct Work {
  int n_units, u_begin, KB, G, cta;
  bool rr;
  Partition part;  // stream-K: which CTA holds which unit
  // stream-K: the range [u_begin, u_begin + n_units) is walked as a list of pieces; piece_start[] are global
  // unit indices, piece_end[] local indices (cumulative lengths).  Today there is one piece: the range front to
  // back.  (Walking the partial tiles at both ends first, so that the launch ends on a whole tile's plain
  // store, was measured 1 us slower on the 192-tile decode GEMM and is not used.)
  int piece_start[3], piece_end[3];
};
__host__ __device__ __forceinline__ void plan_pieces(Work& w) {
  w.piece_start[0] = w.piece_start[1] = w.piece_start[2] = w.u_begin;
  w.piece_end[0] = w.piece_end[1] = w.piece_end[2] = w.n_units;
}
__host__ __device__ __forceinline__ int piece_of(const Work& w, int i) { return i < w.piece_end[0] ? 0 : (i < w.piece_end[1] ? 1 : 2); }
__host__ __device__ __forceinline__ void unit_at(const Work& w, int i, int& tile, int& kb) {
  if (w.rr) {
    const int j = i / w.KB;
    kb = i - j * w.KB;
    tile = w.cta + j * w.G;
  } else {
    const int p = piece_of(w, i);
    const int u = w.piece_start[p] + (i - (p == 0 ? 0 : w.piece_end[p - 1]));
    tile = u / w.KB;
    kb = u - tile * w.KB;
  }
}
// Walks the units one by one without dividing (except once per piece): the TMA producer is a single thread
// whose instruction stream competes with an epilogue warp for issue slots, so its per-K-block arithmetic has
// to stay short.
struct Cursor {
  int tile, kb, tp, tq, i, next_jump;
};
__host__ __device__ __forceinline__ void cursor_seek(const Work& w, int tilesQ, Cursor& c) {
  unit_at(w, c.i, c.tile, c.kb);
  c.tp = c.tile / tilesQ;
  c.tq = c.tile - c.tp * tilesQ;
  c.next_jump = w.rr ? w.n_units : w.piece_end[piece_of(w, c.i)];
}
__host__ __device__ __forceinline__ Cursor cursor_begin(const Work& w, int tilesQ) {
  Cursor c;
  c.i = 0;
  if (w.n_units > 0) cursor_seek(w, tilesQ, c);
  return c;
}
__host__ __device__ __forceinline__ void cursor_next(const Work& w, int tilesQ, Cursor& c) {
  if (++c.i >= w.n_units) return;
  if (c.i == c.next_jump) {  // next piece starts somewhere else
    cursor_seek(w, tilesQ, c);
    return;
  }
  if (++c.kb == w.KB) {
    c.kb = 0;
    const int step = w.rr ? w.G : 1;
    c.tile += step;
    c.tq += step;
    while (c.tq >= tilesQ) {
      c.tq -= tilesQ;
      ++c.tp;
    }
  }
}
__host__ __device__ __forceinline__ bool next_seg(const Work& w, int& i, Seg& s) {
  if (i >= w.n_units) return false;
  int tile, kb;
  unit_at(w, i, tile, kb);
  const int limit = w.rr ? w.n_units : w.piece_end[piece_of(w, i)];
  const int len = (w.KB - kb) < (limit - i) ? (w.KB - kb) : (limit - i);
  s.tile = tile;
  s.kb0 = kb;
  s.kb1 = kb + len;
  i += len;
  return true;
}

// The share of CTA `cta` when `tiles` tiles of KB K blocks are dealt to the first G CTAs of the grid.
__host__ __device__ __forceinline__ Work make_work(int cta, int G, int tiles, int KB, bool rr) {
  Work w;
  const int U = tiles * KB;
  w.part.base = U / G;
  w.part.rem = U % G;
  const Partition& part = w.part;
  w.KB = KB;
  w.G = G;
  w.cta = cta;
  w.rr = rr;
  const bool has = cta < G;
  w.u_begin = has ? part.u0(cta) : 0;
  if (!has) w.n_units = 0;
  else if (rr) w.n_units = ((tiles - cta + G - 1) / G) * KB;
  else w.n_units = part.u0(cta + 1) - w.u_begin;
  plan_pieces(w);
  return w;
}

// Two-shot ownership of token rows: blocks of 16 rows are dealt round-robin to the ranks.
constexpr int OWN_SHIFT = 4, OWN_ROWS = 1 << OWN_SHIFT;
__host__ __device__ __forceinline__ int owner_of(int token, int world, int& local_row) {
  const int b = token >> OWN_SHIFT;
  local_row = ((b / world) << OWN_SHIFT) + (token & (OWN_ROWS - 1));
  return b % world;
}
__host__ __device__ inline int owned_rows(int M, int world, int rank) {
  const int blocks = (M + OWN_ROWS - 1) >> OWN_SHIFT;
  const int mine = (blocks - rank + world - 1) / world;  // blocks rank, rank + world, ...
  if (mine <= 0) return 0;
  const int last_block = rank + (mine - 1) * world;
  const int last_rows = (last_block == blocks - 1) ? M - (last_block << OWN_SHIFT) : OWN_ROWS;
  return (mine - 1) * OWN_ROWS + last_rows;
}

// Row-owner form for few tokens: row t belongs to rank t mod world (balanced for any M), at inbox row t / world.
__host__ __device__ __forceinline__ int owner3_of(int token, int world, int& local_row) {
  local_row = token / world;
  return token - local_row * world;
}
__host__ __device__ __forceinline__ int owned_rows3(int M, int world, int rank) { return (M + world - 1 - rank) / world; }

// ---------------------------------------------------------------------------
// Output of one 32-column chunk held by a warp: thread `lane` has TMEM lane
// (row of the P tile) q*32 + lane and columns c*32 .. c*32+31 (rows of the Q
// tile).
// ---------------------------------------------------------------------------
// silu(gate) * up on bf16-rounded inputs, with the reference's roundings (nanovllm/layers/activation.py:8-11, eager):
// the activation is rounded to bf16 before the product, the product once more by the caller's pack
__device__ __forceinline__ float silu_mul(float gate, float up) {
  return b2::bf16_round(gate / (1.0f + expf(-gate))) * up;
}
// 8 bf16 = 4 (gate, up) pairs -> 4 bf16
__device__ __forceinline__ uint2 silu_mul_pairs(const uint4& w) {
  return make_uint2(b2::pack_bf16(silu_mul(b2::bf16_lo(w.x), b2::bf16_hi(w.x)), silu_mul(b2::bf16_lo(w.y), b2::bf16_hi(w.y))),
                    b2::pack_bf16(silu_mul(b2::bf16_lo(w.z), b2::bf16_hi(w.z)), silu_mul(b2::bf16_lo(w.w), b2::bf16_hi(w.w))));
}

// NC columns (tokens token0 ..) of one feature per lane, features = consecutive lanes.
// Lanes 2i and 2i+1 hold features f and f+1 of the same tokens.  They swap
// halves so that each lane stores a packed (f, f+1) pair: the even lane for
// even columns, the odd lane for odd columns.
template <int NC, int EPI>
__device__ __forceinline__ void emit_feature_lanes(const GemmArgs& a, float (&v)[NC], int feature, int token0, int lane,
                                                   unsigned int parity) {
  if (a.bias != nullptr && feature < a.N) {
    const float b = __uint_as_float(static_cast<uint32_t>(a.bias[feature]) << 16);
#pragma unroll
    for (int j = 0; j < NC; ++j) v[j] += b;
  }
  const int fbase = feature & ~1;
  const bool odd = lane & 1;
#pragma unroll
  for (int j = 0; j < NC; j += 2) {
    const float send = odd ? v[j] : v[j + 1];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
    const int token = token0 + j + (odd ? 1 : 0);
    uint32_t w = odd ? b2::pack_bf16(recv, v[j + 1]) : b2::pack_bf16(v[j], recv);
    if (token < a.M && fbase < a.N) {
      if (EPI == EPI_STORE) {
        if (a.silu_pairs) {  // w = (gate, up) of feature pair fbase / 2
          const float act = silu_mul(b2::bf16_lo(w), b2::bf16_hi(w));
          a.C[token * a.ldc + (fbase >> 1)] = static_cast<uint16_t>(b2::pack_bf16(act, 0.f) & 0xFFFF);
        } else {
          *reinterpret_cast<uint32_t*>(a.C + token * a.ldc + fbase) = w;
        }
      } else if (EPI == EPI_PUSH3) {
        w = b2::scrub_sentinel(w);
        int lrow;
        const int owner = owner3_of(token, a.world, lrow);
        *reinterpret_cast<uint32_t*>(a.inbox[owner] + parity * a.parity_stride + a.rank * a.slot_stride +
                                     (static_cast<size_t>(lrow) * a.N + fbase) * 2) = w;
      } else {
        w = b2::scrub_sentinel(w);
        const size_t off = parity * a.parity_stride + a.rank * a.slot_stride +
                           (static_cast<size_t>(token) * a.N + fbase) * 2;
#pragma unroll
        for (int r = 0; r < B2_MAX_WORLD; ++r)
          if (r < a.world) *reinterpret_cast<uint32_t*>(a.inbox[r] + off) = w;
      }
    }
  }
}

// Token-row epilogue (SWAP = false): a lane holds 32 consecutive features of one token row.  Storing them
// straight from registers would make every store instruction touch 32 different rows with 16 bytes each,
// which wastes NVLink packets when the destination is a peer.  Instead each warp parks up to 4 chunks
// (128 features = 256 bytes per row) in its own 8 KB of shared memory (16-byte pieces XOR-swizzled by row)
// and then writes whole 256-byte row segments, two rows per instruction.
constexpr int STAGE_ROW_BYTES = 256;
constexpr int STAGING_BYTES_PER_WARP = 32 * STAGE_ROW_BYTES;

__device__ __forceinline__ void stage_row_chunk(const GemmArgs& a, unsigned char* wbuf, int lane, int slot, float (&v)[32], int feature0,
                                                bool scrub) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int feature = feature0 + g * 8;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = v[g * 8 + e];
    if (a.bias != nullptr && feature < a.N) {
      const uint4 bv = *reinterpret_cast<const uint4*>(a.bias + feature);
      f[0] += b2::bf16_lo(bv.x); f[1] += b2::bf16_hi(bv.x); f[2] += b2::bf16_lo(bv.y); f[3] += b2::bf16_hi(bv.y);
      f[4] += b2::bf16_lo(bv.z); f[5] += b2::bf16_hi(bv.z); f[6] += b2::bf16_lo(bv.w); f[7] += b2::bf16_hi(bv.w);
    }
    uint4 w = make_uint4(b2::pack_bf16(f[0], f[1]), b2::pack_bf16(f[2], f[3]), b2::pack_bf16(f[4], f[5]), b2::pack_bf16(f[6], f[7]));
    if (scrub) {
      w.x = b2::scrub_sentinel(w.x); w.y = b2::scrub_sentinel(w.y);
      w.z = b2::scrub_sentinel(w.z); w.w = b2::scrub_sentinel(w.w);
    }
    const int piece = slot * 4 + g;
    *reinterpret_cast<uint4*>(wbuf + lane * STAGE_ROW_BYTES + ((piece ^ (lane & 15)) << 4)) = w;
  }
}

template <int EPI>
__device__ __forceinline__ void flush_rows(const GemmArgs& a, unsigned char* wbuf, int lane, int token0, int feature0, int npieces,
                                           unsigned int parity) {
  __syncwarp();
  const int piece = lane & 15;
  const int feature = feature0 + piece * 8;
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int row = it * 2 + (lane >> 4);
    const int token = token0 + row;
    if (piece < npieces && token < a.M && feature < a.N) {
      const uint4 w = *reinterpret_cast<const uint4*>(wbuf + row * STAGE_ROW_BYTES + ((piece ^ (row & 15)) << 4));
      if (EPI == EPI_STORE) {
        if (a.silu_pairs) *reinterpret_cast<uint2*>(a.C + token * a.ldc + (feature >> 1)) = silu_mul_pairs(w);
        else *reinterpret_cast<uint4*>(a.C + token * a.ldc + feature) = w;
      } else if (EPI == EPI_PUSH2) {
        int lrow;
        const int owner = owner_of(token, a.world, lrow);
        *reinterpret_cast<uint4*>(a.inbox[owner] + parity * a.parity_stride + a.rank * a.slot_stride +
                                  (static_cast<size_t>(lrow) * a.N + feature) * 2) = w;
      } else if (EPI == EPI_PUSH3) {
        int lrow;
        const int owner = owner3_of(token, a.world, lrow);
        *reinterpret_cast<uint4*>(a.inbox[owner] + parity * a.parity_stride + a.rank * a.slot_stride +
                                  (static_cast<size_t>(lrow) * a.N + feature) * 2) = w;
      } else {
        const size_t off = parity * a.parity_stride + a.rank * a.slot_stride + (static_cast<size_t>(token) * a.N + feature) * 2;
#pragma unroll
        for (int r = 0; r < B2_MAX_WORLD; ++r)
          if (r < a.world) *reinterpret_cast<uint4*>(a.inbox[r] + off) = w;
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------
// Sampler fused into the LM-head epilogue.
// The reference draws token = argmax_i softmax(logit / T)_i / E_i with E_i ~ Exp(1)
// (nanovllm/layers/sampler.py:9-11).  The softmax denominator is the same for every i of a row and log is
// monotone, so the same token is argmax_i (logit_i / T - log E_i): no pass over the whole row is needed,
// each rank can scan its own slice of the vocabulary, and only (best score, vocab id) per row is exchanged.
// E_i comes from Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed by
// the caller's seed, with counter (vocab id, token row / 4, call number, tag): the draw for an element depends
// on nothing but those, so it is the same for every tensor-parallel split and can be regenerated on the host.
// ---------------------------------------------------------------------------
constexpr uint32_t SAMPLE_TAG = 0x53414D50u;

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0], p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0, n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
    c[1] = static_cast<uint32_t>(p1);
    c[3] = static_cast<uint32_t>(p0);
    c[0] = n0;
    c[2] = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}
// 23 random bits -> u in (0, 1), both ends excluded and every value exact in fp32; E = -log u is Exp(1)
__device__ __forceinline__ float gumbel_from_bits(uint32_t x) {
  const float u = (static_cast<float>(x >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
  return -logf(-logf(u));
}
// unsigned order of the key = (score ascending, then vocab id descending): max picks the best score, lowest id on ties
__host__ __device__ __forceinline__ unsigned long long sample_key(uint32_t score_bits, uint32_t vocab_id) {
  const uint32_t ord = (score_bits & 0x80000000u) ? ~score_bits : (score_bits | 0x80000000u);
  return (static_cast<unsigned long long>(ord) << 32) | (0xFFFFFFFFu - vocab_id);
}

// One 32-token chunk of one vocabulary entry per lane (feature-lane layout).  The 32 x 32 keys of the warp are
// reduced over the lanes by a halving exchange (31 shuffles of a key instead of 32 x 5): afterwards lane l holds
// the best key of token token0 + l among the warp's 32 vocabulary entries, and merges it into the CTA's table.
__device__ __forceinline__ void sample_feature_lanes(const GemmArgs& a, float (&v)[32], int feature, int token0, int lane,
                                                     unsigned int call, unsigned long long* cta_best) {
  const bool live = feature < a.N;
  const uint32_t vocab_id = static_cast<uint32_t>(a.vocab_offset + feature);
  const float bias = (a.bias != nullptr && live) ? __uint_as_float(static_cast<uint32_t>(a.bias[feature]) << 16) : 0.f;
  unsigned long long k[32];
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += 4) {
    uint32_t r[4] = {vocab_id, static_cast<uint32_t>(token0 + j0) >> 2, call, SAMPLE_TAG};
    if (a.temperatures != nullptr) philox4x32_10(r, static_cast<uint32_t>(a.seed), static_cast<uint32_t>(a.seed >> 32));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int token = token0 + j0 + i;
      float z = b2::bf16_round(v[j0 + i] + bias);  // the logit as the unfused path stores it
      if (a.temperatures != nullptr && token < a.M) z = z / __ldg(a.temperatures + token) + gumbel_from_bits(r[i]);
      k[j0 + i] = (live && token < a.M) ? sample_key(__float_as_uint(z), vocab_id) : 0ull;
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int j = 0; j < o; ++j) {
      const unsigned long long send = upper ? k[j] : k[j + o];
      const unsigned long long keep = upper ? k[j + o] : k[j];
      const unsigned long long recv = __shfl_xor_sync(0xffffffffu, send, o);
      k[j] = keep > recv ? keep : recv;
    }
  }
  if (k[0] != 0ull) atomicMax(cta_best + token0 + lane, k[0]);
}

// One 32-column chunk c of a tile leaves the registers.  Feature-lane layout (SWAP): stored at once.
// Token-row layout: parked in the warp's staging buffer; every fourth chunk (and the tile's last) flushes.
template <int BN, bool SWAP, int EPI>
__device__ __forceinline__ void emit_chunk(const GemmArgs& a, float (&v)[32], int p_row, int q_tile0, int c, int lane, unsigned int parity,
                                           unsigned char* wbuf, unsigned int sample_call, unsigned long long* cta_best) {
  if constexpr (EPI == EPI_SAMPLE) {
    static_assert(SWAP, "the fused sampler needs the feature-lane layout");
    sample_feature_lanes(a, v, p_row, q_tile0 + c * 32, lane, sample_call, cta_best);
  } else if (SWAP) {
    emit_feature_lanes<32, EPI>(a, v, p_row, q_tile0 + c * 32, lane, parity);
  } else {
    stage_row_chunk(a, wbuf, lane, c & 3, v, q_tile0 + c * 32, is_push(EPI));
    if ((c & 3) == 3 || c == BN / 32 - 1)
      flush_rows<EPI>(a, wbuf, lane, p_row - lane, q_tile0 + (c & ~3) * 32, ((c & 3) + 1) * 4, parity);
  }
}

// ---------------------------------------------------------------------------
// Reduce phase of the fused row-parallel call: one CTA per token row.
// S = number of source ranks.  The loads of a row (residual, every source's
// partial, norm weight) are issued together, G vectors at a time, so that a
// thread pays one memory round trip per group instead of one per vector.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  acc[0] += b2::bf16_lo(v.x); acc[1] += b2::bf16_hi(v.x); acc[2] += b2::bf16_lo(v.y); acc[3] += b2::bf16_hi(v.y);
  acc[4] += b2::bf16_lo(v.z); acc[5] += b2::bf16_hi(v.z); acc[6] += b2::bf16_lo(v.w); acc[7] += b2::bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  return make_uint4(b2::pack_bf16(f[0], f[1]), b2::pack_bf16(f[2], f[3]), b2::pack_bf16(f[4], f[5]), b2::pack_bf16(f[6], f[7]));
}

// FORM_ALL   (one-shot): every rank reduces every row; outputs go to normed_out / residual_out.
// FORM_BLOCKS(two-shot): this rank reduces only the rows it owns (16-row blocks, round-robin); a finished row
//                        goes into every rank's output buffer, the new residual stays with the owner.
// FORM_OWNER (few tokens): this rank reduces the rows t with t mod world == rank; the finished row and the new
//                        residual row go into every rank's landing buffer (data-as-flag: sentinel scrubbed).
// Returns the rows finished.
enum { FORM_ALL = 0, FORM_BLOCKS = 1, FORM_OWNER = 2 };

template <int FORM>
__device__ __forceinline__ void store_finished(const GemmArgs& a, unsigned int parity, int plane, size_t elem_off, uint4 y) {
  if (FORM == FORM_BLOCKS) {
#pragma unroll
    for (int r = 0; r < B2_MAX_WORLD; ++r)
      if (r < a.world) *reinterpret_cast<uint4*>(a.inbox[r] + a.out_off + elem_off * 2) = y;
  } else if (FORM == FORM_OWNER) {
    y.x = b2::scrub_sentinel(y.x); y.y = b2::scrub_sentinel(y.y);
    y.z = b2::scrub_sentinel(y.z); y.w = b2::scrub_sentinel(y.w);
    const size_t off = a.land_off + parity * a.land_parity_stride + plane * a.land_plane_stride + elem_off * 2;
#pragma unroll
    for (int r = 0; r < B2_MAX_WORLD; ++r)
      if (r < a.world) *reinterpret_cast<uint4*>(a.inbox[r] + off) = y;
  } else {
    *reinterpret_cast<uint4*>((plane == 0 ? a.normed_out : a.residual_out) + elem_off) = y;
  }
}

template <int S, int FORM>
__device__ __forceinline__ int reduce_rows(const GemmArgs& a, unsigned int parity, float* red, volatile int* gave_up) {
  // vectors in flight together: G * S loads of 16 bytes (a 4096-wide row at 8 ranks is one batch of 24 loads per thread)
  constexpr int G = S >= 8 ? 3 : (S == 4 ? 3 : MAX_ROW_VECS);
  constexpr bool TWO = FORM == FORM_BLOCKS;
  const int nvec = a.N >> 3;
  const int tid = threadIdx.x;
  const bool with_norm = a.norm_w != nullptr;
  unsigned char* my = a.inbox[a.rank] + parity * a.parity_stride;
  const uint4 sentinel = make_uint4(B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32);
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  // Every CTA takes rows blockIdx, blockIdx + grid, ... once its GEMM work is done.  (Setting CTAs aside that only
  // reduce, following the GEMM's sweep over the rows, was measured and lost: a CTA reduces a row in about 5 us,
  // latency-bound, so few reducers cannot keep up and many cost the GEMM its SMs.)
  int n_rows = a.M, row0 = blockIdx.x, row_step = gridDim.x;
  if (TWO) n_rows = owned_rows(a.M, a.world, a.rank);
  if (FORM == FORM_OWNER) n_rows = owned_rows3(a.M, a.world, a.rank);
  int rows_done = 0;
  for (int row = row0; row < n_rows; row += row_step, ++rows_done) {
    float acc[MAX_ROW_VECS][8];
    float ss = 0.f;
    const size_t row_off = static_cast<size_t>(row) * a.N;  // row inside the inbox
    // row of the [M, N] tensors: two-shot owners hold the 16-row blocks rank, rank + world, ...; the owner form rows rank, rank + world, ...
    const int token = TWO ? ((((row >> OWN_SHIFT) * a.world + a.rank) << OWN_SHIFT) + (row & (OWN_ROWS - 1)))
                          : (FORM == FORM_OWNER ? row * a.world + a.rank : row);
    const size_t out_off = static_cast<size_t>(token) * a.N;
#pragma unroll
    for (int g0 = 0; g0 < MAX_ROW_VECS; g0 += G) {
      if (tid + g0 * NUM_THREADS >= nvec) break;
      uint4 resv[G];
      uint4 val[G][S];
      // residual first: it does not depend on the partials
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int v = tid + (g0 + i) * NUM_THREADS;
        resv[i] = (with_norm && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(a.residual_in + out_off + v * 8)) : zero4;
      }
      bool pending = true;
      uint64_t t0 = 0;
      for (uint32_t spin = 0; pending; ++spin) {
        pending = false;
#pragma unroll
        for (int i = 0; i < G; ++i) {
          const int v = tid + (g0 + i) * NUM_THREADS;
          if (v < nvec) {
#pragma unroll
            for (int s = 0; s < S; ++s) val[i][s] = b2::ld_volatile_v4(my + s * a.slot_stride + (row_off + v * 8) * 2);
          }
        }
#pragma unroll
        for (int i = 0; i < G; ++i) {
          const int v = tid + (g0 + i) * NUM_THREADS;
          if (v < nvec) {
#pragma unroll
            for (int s = 0; s < S; ++s) pending |= b2::has_sentinel(val[i][s]);
          }
        }
        if (pending && (spin & 0x3F) == 0x3F) {
          // one expired wait ends every later wait of this CTA at once
          if (*gave_up) break;
          if (t0 == 0) t0 = b2::globaltimer_ns();
          else if (b2::time_limit_passed(t0, a.timeout_ns)) {
            *gave_up = 1;
            b2::report_timeout(a.status, B2_WAIT_PARTIALS);
            break;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int v = tid + (g0 + i) * NUM_THREADS;
        if (v < nvec) {
          const size_t eoff = row_off + v * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g0 + i][e] = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) {
            add8(acc[g0 + i], val[i][s]);
            *reinterpret_cast<uint4*>(my + s * a.slot_stride + eoff * 2) = sentinel;  // consumed
          }
          if (with_norm) {
            add8(acc[g0 + i], resv[i]);
            if (FORM == FORM_OWNER) store_finished<FORM_OWNER>(a, parity, 1, out_off + v * 8, pack8f(acc[g0 + i]));
            else *reinterpret_cast<uint4*>(a.residual_out + out_off + v * 8) = pack8f(acc[g0 + i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += acc[g0 + i][e] * acc[g0 + i][e];
          } else {
            store_finished<FORM>(a, parity, 0, out_off + v * 8, pack8f(acc[g0 + i]));
          }
        }
      }
    }
    if (!with_norm) continue;  // plain all-reduce: done with this row (uniform across the CTA)
    // the norm weights travel while the row's sum of squares is being combined
    uint4 wv[MAX_ROW_VECS];
#pragma unroll
    for (int it = 0; it < MAX_ROW_VECS; ++it) {
      const int v = tid + it * NUM_THREADS;
      wv[it] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(a.norm_w + v * 8)) : zero4;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();  // red[] free again
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < NUM_THREADS / 32; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / static_cast<float>(a.N) + a.eps);
#pragma unroll
    for (int it = 0; it < MAX_ROW_VECS; ++it) {
      const int v = tid + it * NUM_THREADS;
      if (v < nvec) {
        float o[8];
        o[0] = b2::bf16_round(acc[it][0] * rstd) * b2::bf16_lo(wv[it].x); o[1] = b2::bf16_round(acc[it][1] * rstd) * b2::bf16_hi(wv[it].x);
        o[2] = b2::bf16_round(acc[it][2] * rstd) * b2::bf16_lo(wv[it].y); o[3] = b2::bf16_round(acc[it][3] * rstd) * b2::bf16_hi(wv[it].y);
        o[4] = b2::bf16_round(acc[it][4] * rstd) * b2::bf16_lo(wv[it].z); o[5] = b2::bf16_round(acc[it][5] * rstd) * b2::bf16_hi(wv[it].z);
        o[6] = b2::bf16_round(acc[it][6] * rstd) * b2::bf16_lo(wv[it].w); o[7] = b2::bf16_round(acc[it][7] * rstd) * b2::bf16_hi(wv[it].w);
        store_finished<FORM>(a, parity, 0, out_off + v * 8, pack8f(o));
      }
    }
  }
  return rows_done;
}

// Owner form, last phase: every (plane, row, 16-byte vector) of the landing buffer is copied into the caller's
// tensors once it has landed (data-as-flag: the vector holds the sentinel until then) and the sentinel is put back.
// The items are dealt to all threads of the grid, LAND_BATCH loads in flight per thread.
constexpr int LAND_BATCH = 4;
__device__ __forceinline__ void collect_landed_rows(const GemmArgs& a, unsigned int parity, volatile int* gave_up) {
  const int nvec = a.N >> 3;
  const int planes = a.norm_w != nullptr ? 2 : 1;
  const int64_t per_plane = static_cast<int64_t>(a.M) * nvec;
  const int64_t total = per_plane * planes;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * NUM_THREADS;
  unsigned char* land = a.inbox[a.rank] + a.land_off + parity * a.land_parity_stride;
  const uint4 sentinel = make_uint4(B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32, B2_SENTINEL32);
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * NUM_THREADS + threadIdx.x; base < total; base += stride * LAND_BATCH) {
    uint4 val[LAND_BATCH];
    unsigned char* src[LAND_BATCH];
    uint16_t* dst[LAND_BATCH];
    bool todo[LAND_BATCH];
#pragma unroll
    for (int i = 0; i < LAND_BATCH; ++i) {
      const int64_t idx = base + i * stride;
      todo[i] = idx < total;
      const int plane = (todo[i] && idx >= per_plane) ? 1 : 0;
      const int64_t e = (todo[i] ? idx - plane * per_plane : 0) * 8;  // element offset inside the plane
      src[i] = land + plane * a.land_plane_stride + e * 2;
      dst[i] = (plane == 0 ? a.normed_out : a.residual_out) + e;
    }
    bool pending = true;
    uint64_t t0 = 0;
    for (uint32_t spin = 0; pending; ++spin) {
      pending = false;
#pragma unroll
      for (int i = 0; i < LAND_BATCH; ++i)
        if (todo[i]) val[i] = b2::ld_volatile_v4(src[i]);
#pragma unroll
      for (int i = 0; i < LAND_BATCH; ++i) {
        if (todo[i]) {
          if (b2::has_sentinel(val[i])) {
            pending = true;
          } else {
            *reinterpret_cast<uint4*>(dst[i]) = val[i];
            *reinterpret_cast<uint4*>(src[i]) = sentinel;
            todo[i] = false;
          }
        }
      }
      if (pending && (spin & 0x3F) == 0x3F) {
        if (*gave_up) return;
        if (t0 == 0) t0 = b2::globaltimer_ns();
        else if (b2::time_limit_passed(t0, a.timeout_ns)) {
          *gave_up = 1;
          b2::report_timeout(a.status, B2_WAIT_ROWS);
          return;
        }
      }
    }
  }
}

__device__ __forceinline__ void stamp(const GemmArgs& a, int slot) {
  if (a.trace != nullptr) {
    unsigned long long* t = a.trace + (static_cast<size_t>(blockIdx.x) * 8 + slot) * 2;
    t[0] = static_cast<unsigned long long>(clock64());
    t[1] = b2::globaltimer_ns();
  }
}

// What follows the GEMM part of a fused row-parallel launch: the reduce phase (one-shot: all rows; two-shot:
// owned rows, then the arrival count of finished rows) and the advance of the launch parity.
template <int EPI>
__device__ __forceinline__ void fused_tail(const GemmArgs& a, unsigned int parity, float* red, volatile int* abort_flag, int aborted) {
  if (threadIdx.x == 0) stamp(a, 5);
  if (is_push(EPI)) {
    // Every partial row of this CTA is on its way: from here on the CTA only waits for data, so the next kernel's CTAs
    // may take the SMs that are free.  (Released at set-up instead, they could occupy SMs before all CTAs of this
    // grid are resident, while the resident ones spin on rows the missing ones have yet to produce.)
// Row-owner form: every rank waits for every other rank inside the same launch, so a store to a peer that lingers in
    // a write buffer until the kernel ends would never leave: push the partial rows out before waiting for anything.
    if (EPI == EPI_PUSH3) __threadfence_system();
        if (threadIdx.x == 0) b2::pdl_launch_dependents();
    if (!aborted) {
      if (EPI == EPI_PUSH) {
        switch (a.world) {
          case 1: reduce_rows<1, FORM_ALL>(a, parity, red, abort_flag); break;
          case 2: reduce_rows<2, FORM_ALL>(a, parity, red, abort_flag); break;
          case 4: reduce_rows<4, FORM_ALL>(a, parity, red, abort_flag); break;
          default: reduce_rows<8, FORM_ALL>(a, parity, red, abort_flag); break;
        }
      } else if (EPI == EPI_PUSH3) {
        switch (a.world) {
          case 1: reduce_rows<1, FORM_OWNER>(a, parity, red, abort_flag); break;  // one rank owns every row (the mechanism on a single GPU)
          case 2: reduce_rows<2, FORM_OWNER>(a, parity, red, abort_flag); break;
          case 4: reduce_rows<4, FORM_OWNER>(a, parity, red, abort_flag); break;
          default: reduce_rows<8, FORM_OWNER>(a, parity, red, abort_flag); break;
        }
        __threadfence_system();  // the finished rows leave for the peers now (see above)
        if (threadIdx.x == 0) stamp(a, 4);  // owned rows finished and sent (overwrites "epilogue done": the GEMM part's end is stamp 5)
        collect_landed_rows(a, parity, abort_flag);
      } else {
        int rows_done = 0;
        switch (a.world) {
          case 2: rows_done = reduce_rows<2, FORM_BLOCKS>(a, parity, red, abort_flag); break;
          case 4: rows_done = reduce_rows<4, FORM_BLOCKS>(a, parity, red, abort_flag); break;
          default: rows_done = reduce_rows<8, FORM_BLOCKS>(a, parity, red, abort_flag); break;
        }
        // the finished rows must be visible on every GPU before their count is
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0 && rows_done > 0) {
          for (int r = 0; r < a.world; ++r)
            if (r != a.rank)
              asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned int*>(a.inbox[r] + a.rowcnt_off) + parity), "r"(static_cast<unsigned int>(rows_done)) : "memory");
        }
        // one CTA holds the launch open until the rows owned elsewhere have all arrived here
        if (blockIdx.x == 0 && threadIdx.x == 0) {
          const int mine = owned_rows(a.M, a.world, a.rank);
          const unsigned int expect = static_cast<unsigned int>(a.M - mine);
          unsigned int* cnt = reinterpret_cast<unsigned int*>(a.inbox[a.rank] + a.rowcnt_off) + parity;
          const uint64_t t0 = b2::globaltimer_ns();
          for (uint32_t spin = 0;; ++spin) {
            unsigned int got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(cnt) : "memory");
            if (got >= expect) break;
            if ((spin & 0xFF) == 0xFF && b2::time_limit_passed(t0, a.timeout_ns)) {
              b2::report_timeout(a.status, B2_WAIT_ROWS);
              break;
            }
          }
          *reinterpret_cast<volatile unsigned int*>(cnt) = 0;  // next used two launches from now, after every peer has seen this launch end
        }
      }
    }
    // the last CTA to finish advances the launch parity for the next call
    __syncthreads();
    if (threadIdx.x == 0) {
      stamp(a, 6);
      __threadfence();
      const unsigned int prev = atomicAdd(&a.dstate->rowpar_done, 1u);
      if (prev == gridDim.x - 1) {
        a.dstate->rowpar_done = 0;
        a.dstate->rowpar_seq += 1;
        __threadfence();
      }
    }
  }
}

// The CTA's table of best keys per token row (fused sampler only; other epilogues carry no such array)
template <int EPI>
struct SampleTable {
  __device__ static __forceinline__ unsigned long long* get() { return nullptr; }
};
template <>
struct SampleTable<EPI_SAMPLE> {
  __device__ static __forceinline__ unsigned long long* get() {
    __shared__ unsigned long long table[256];
    return table;
  }
};

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int BN, bool SWAP, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, const GemmArgs a) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = b2::smem_u32(smem_raw);
  unsigned char* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  const uint32_t smem_base = b2::smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  const uint32_t bar_full = b2::smem_u32(bars);
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  constexpr int ACC = C::ACC;
  const uint32_t bar_tempty = bar_tfull + ACC * 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float red[NUM_THREADS / 32];
  unsigned long long* const cta_best = SampleTable<EPI>::get();
  unsigned int sample_call = 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int KB = a.kblocks;
  const int tiles = a.tilesP * a.tilesQ;
  const bool has_gemm = cta < a.gemm_ctas;
  const Work work = make_work(cta, a.gemm_ctas, tiles, KB, a.round_robin != 0);

  if (threadIdx.x == 0) {
    stamp(a, 7);
    b2::tma_prefetch_desc(&tmP);
    b2::tma_prefetch_desc(&tmQ);
    for (int s = 0; s < STAGES; ++s) {
      b2::mbar_init(bar_full + s * 8, 1);
      b2::mbar_init(bar_empty + s * 8, 1);
    }
    for (int i = 0; i < ACC; ++i) {
      b2::mbar_init(bar_tfull + i * 8, 1);
      b2::mbar_init(bar_tempty + i * 8, 4);
    }
    *abort_flag = 0;
    b2::mbar_fence_init();
  }
  if constexpr (EPI == EPI_SAMPLE)
    for (int t = threadIdx.x; t < 256; t += NUM_THREADS) cta_best[t] = 0ull;
  if (warp == 1 && has_gemm) {
    b2::tmem_alloc(b2::smem_u32(tmem_slot), C::TMEM_COLS);
    b2::tmem_relinquish();
  }
  b2::tc_fence_before();
  __syncthreads();
  b2::tc_fence_after();
  const uint32_t tmem_base = has_gemm ? *tmem_slot : 0;
  // The next kernel in the stream may start its own set-up from now on - unless this launch is a fused row-parallel
  // call: its CTAs later wait for rows that other CTAs of the same grid (and of the peers' grids) produce, so the
  // dependents are released only once every CTA has delivered its part (fused_tail), when nothing of this grid
  // needs an SM any more.
  if (threadIdx.x == 0 && !is_push(EPI)) b2::pdl_launch_dependents();
  if (threadIdx.x == 0) stamp(a, 0);
  unsigned int parity = 0;

  if (has_gemm) {
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        const uint64_t polP = SWAP ? b2::kEvictFirst : b2::kEvictNormal;
        const uint64_t polQ = SWAP ? b2::kEvictLast : b2::kEvictNormal;
        const int n_units = work.n_units;
        const int pre = n_units < STAGES ? n_units : STAGES;
        // The weight tiles of the first stages depend on no earlier kernel: fetch them before the
        // dependency wait, so that they are in flight (or landed) when the activations become valid.
        Cursor cw = cursor_begin(work, a.tilesQ);
        for (int i = 0; i < pre; ++i) {
          const uint32_t fb = bar_full + i * 8;
          b2::mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
          const uint32_t dst = smem_base + i * C::STAGE_BYTES;
          if (SWAP) b2::tma_load_2d(dst, &tmP, fb, cw.kb * BK, cw.tp * BM, polP);
          else b2::tma_load_2d(dst + C::P_BYTES, &tmQ, fb, cw.kb * BK, cw.tq * BN, polQ);
          cursor_next(work, a.tilesQ, cw);
        }
        b2::pdl_wait();
        stamp(a, 3);
        Cursor cx = cursor_begin(work, a.tilesQ);
        for (int i = 0; i < pre; ++i) {
          const uint32_t fb = bar_full + i * 8;
          const uint32_t dst = smem_base + i * C::STAGE_BYTES;
          if (SWAP) b2::tma_load_2d(dst + C::P_BYTES, &tmQ, fb, cx.kb * BK, cx.tq * BN, polQ);
          else b2::tma_load_2d(dst, &tmP, fb, cx.kb * BK, cx.tp * BM, polP);
          cursor_next(work, a.tilesQ, cx);
        }
        int stage = pre == STAGES ? 0 : pre;
        uint32_t phase = pre == STAGES ? 1 : 0;
        for (int i = pre; i < n_units; ++i) {  // cx now stands at unit `pre`
          if (!b2::mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_EMPTY)) break;
          const uint32_t fb = bar_full + stage * 8;
          b2::mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
          const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
          b2::tma_load_2d(dst, &tmP, fb, cx.kb * BK, cx.tp * BM, polP);
          b2::tma_load_2d(dst + C::P_BYTES, &tmQ, fb, cx.kb * BK, cx.tq * BN, polQ);
          cursor_next(work, a.tilesQ, cx);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        constexpr uint32_t idesc = b2::umma_idesc_bf16(BN);
        // The first stage cannot fill before the earlier kernels have completed (the activations are fetched after the
        // producer's dependency wait): wait for them here, so that the pipeline's time limit measures the pipeline
        // alone and not an earlier kernel that is itself waiting for a peer.
        b2::pdl_wait();
        int stage = 0;
        uint32_t phase = 0;
        int u = 0, seg = 0;
        Seg s;
        bool ok = true;
        while (ok && next_seg(work, u, s)) {
          const int acc = seg % ACC;
          const uint32_t use = static_cast<uint32_t>(seg / ACC);  // how often this accumulator was used before
          if (!b2::mbar_wait(bar_tempty + acc * 8, (use & 1) ^ 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_TMEM_EMPTY)) break;
          b2::tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = s.kb0; kb < s.kb1; ++kb) {
            if (!b2::mbar_wait(bar_full + stage * 8, phase, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_FULL)) { ok = false; break; }
            if (seg == 0 && kb == s.kb0) stamp(a, 1);
            b2::tc_fence_after();
            const uint32_t sp = smem_base + stage * C::STAGE_BYTES;
            const uint64_t dp = b2::umma_smem_desc(sp);
            const uint64_t dq = b2::umma_smem_desc(sp + C::P_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // advancing K by 16 elements = 32 bytes inside the 128-byte swizzle row
              b2::umma_bf16(d_tmem, dp + 2 * k, dq + 2 * k, idesc, (kb > s.kb0 || k > 0) ? 1u : 0u);
            }
            b2::umma_commit(bar_empty + stage * 8);  // stage reusable once these MMAs have read it
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          b2::umma_commit(bar_tfull + acc * 8);
          ++seg;
        }
        stamp(a, 2);
      }
    } else {
      // ---------------- epilogue warps ----------------
      const int q = warp & 3;  // TMEM lane quadrant this warp may read
      unsigned char* wbuf = smem + STAGES * C::STAGE_BYTES + 256 + q * STAGING_BYTES_PER_WARP;  // token-row layout only
      b2::pdl_wait();
      if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
      if constexpr (EPI == EPI_SAMPLE) sample_call = *reinterpret_cast<volatile unsigned int*>(&a.dstate->sample_seq);
      int u = 0, seg = 0;
      Seg s;
      while (next_seg(work, u, s)) {
        const int acc = seg % ACC;
        const uint32_t use = static_cast<uint32_t>(seg / ACC);
        if (!b2::mbar_wait(bar_tfull + acc * 8, use & 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_TMEM_FULL)) break;
        b2::tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
        const int tp = s.tile / a.tilesQ, tq = s.tile - tp * a.tilesQ;
        const int p_row = tp * BM + q * 32 + lane;
        const bool whole = (s.kb0 == 0 && s.kb1 == KB);
        if (whole) {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            b2::tmem_ld_32x32(taddr + c * 32, r);
            b2::tc_wait_ld();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            emit_chunk<BN, SWAP, EPI>(a, v, p_row, tq * BN, c, lane, parity, wbuf, sample_call, cta_best);
          }
        } else {
          // This CTA holds only part of the tile's K range.  Every contributor adds its part into the
          // tile's fp32 accumulation slot (vector reductions that complete in L2; nobody waits for them);
          // the contributor that arrives last at the tile's counter reads the sum once, puts the slot
          // back to zero for the next launch, and writes the output.  The slot of a split tile is indexed
          // by its first contributor, which is unique among split tiles.
          const int c_first = work.part.cta_of(s.tile * KB), c_last = work.part.cta_of(s.tile * KB + KB - 1);
          float* slot = a.ws + (static_cast<size_t>(c_first) * 4 + q) * (BN * 32) + lane * 4;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            b2::tmem_ld_32x32(taddr + c * 32, r);
            b2::tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(slot + (c * 8 + j) * 128), "f"(__uint_as_float(r[4 * j])),
                           "f"(__uint_as_float(r[4 * j + 1])), "f"(__uint_as_float(r[4 * j + 2])), "f"(__uint_as_float(r[4 * j + 3]))
                           : "memory");
          }
          __threadfence();
          __syncwarp();
          int old = 0;
          if (lane == 0) old = atomicAdd(a.counters + s.tile * 4 + q, 1);
          old = __shfl_sync(0xffffffffu, old, 0);
          if (old == c_last - c_first) {
            __threadfence();
            if (lane == 0) a.counters[s.tile * 4 + q] = 0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 t;
                asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "l"(slot + (c * 8 + j) * 128) : "memory");
                v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(slot + (c * 8 + j) * 128) = make_float4(0.f, 0.f, 0.f, 0.f);
              emit_chunk<BN, SWAP, EPI>(a, v, p_row, tq * BN, c, lane, parity, wbuf, sample_call, cta_best);
            }
          }
        }
        b2::tc_fence_before();
        __syncwarp();
        if (lane == 0) b2::mbar_arrive(bar_tempty + acc * 8);
        ++seg;
      }
      if (warp == 2 && lane == 0) stamp(a, 4);
    }
  }

  // ---- all roles meet; tensor memory goes back ------------------------------
  b2::pdl_wait();
  if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
  __syncwarp();
  b2::tc_fence_before();
  __syncthreads();
  b2::tc_fence_after();
  const int aborted = *abort_flag;
  if (aborted) {
    // let bulk copies that may still be in flight land before the CTA leaves
    for (int i = 0; i < 100; ++i) __nanosleep(2000);
    if (threadIdx.x == 0) b2::report_timeout(a.status, aborted);
  }
  if (warp == 1 && has_gemm) b2::tmem_dealloc(tmem_base, C::TMEM_COLS);
  if constexpr (EPI == EPI_SAMPLE) {
    // the CTA's best key per token row joins the launch-wide table (feature-lane layout: one token tile, row = token)
    for (int t = threadIdx.x; t < BN; t += NUM_THREADS)
      if (t < a.M && cta_best[t] != 0ull) atomicMax(a.sample_keys + t, cta_best[t]);
  }

  fused_tail<EPI>(a, parity, red, abort_flag, aborted);
}

// ---------------------------------------------------------------------------
// Few tokens, few output tiles (decode): one thread-block cluster per 128-feature output tile.
// The S CTAs of a cluster split the tile's K range; every CTA accumulates its part in tensor memory,
// then the parts are combined through distributed shared memory: the accumulator's 4-column groups are
// dealt round-robin to the CTAs of the cluster, each CTA receives the other CTAs' parts of its groups
// in its own shared memory, sums them after one cluster barrier, and writes its share of the output
// as whole 256-byte token rows.  No global-memory round trip and no atomics on the critical path.
// Feature-lane layout only (weights on the 128-row MMA side); up to 256 tokens as token tiles of BN <= 64, one cluster each.
// ---------------------------------------------------------------------------
template <int BN>
struct CfgCluster {
  static constexpr uint32_t P_BYTES = BM * BK * 2;
  static constexpr uint32_t Q_BYTES = BN * BK * 2;
  static constexpr uint32_t STAGE_BYTES = P_BYTES + Q_BYTES;
  static constexpr int GROUPS = BN / 4;                                 // 4-column groups of the accumulator
  static constexpr uint32_t RED_BYTES = (GROUPS + 8) * BM * 16;         // [source CTA][local group][feature][4] fp32
  static constexpr uint32_t OUT_BYTES = BN * BM * 2;                    // [token][feature] bf16 staging of the output
  static constexpr int STAGES_RAW = (200704 - RED_BYTES - OUT_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + RED_BYTES + OUT_BYTES;
  static_assert(STAGES >= 3, "too little shared memory left for the operand pipeline");
  static_assert(SMEM_BYTES <= 232448, "more shared memory than an SM has");
};

template <int BN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, const GemmArgs a) {
  using C = CfgCluster<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_addr = b2::smem_u32(smem_raw);
  unsigned char* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  const uint32_t smem_base = b2::smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  const uint32_t bar_full = b2::smem_u32(bars);
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned char* red_buf = smem + STAGES * C::STAGE_BYTES + 256;
  unsigned char* out_buf = red_buf + C::RED_BYTES;
  __shared__ float red[NUM_THREADS / 32];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = static_cast<int>(b2::cluster_nctarank());
  const int crank = static_cast<int>(b2::cluster_ctarank());
  // the output tile of this cluster: features [tile * 128, +128) of the tokens [tok0, tok0 + BN); the token tiles of one
  // feature tile belong to consecutive clusters, so that its weight tiles are read from DRAM once and from L2 after that
  const int ct = blockIdx.x / S;
  const int tile = ct / a.tilesQ;
  const int tok0 = (ct - tile * a.tilesQ) * BN;
  const int KB = a.kblocks;
  const int kb_base = KB / S, kb_rem = KB % S;
  const int kb0 = crank * kb_base + min(crank, kb_rem);
  const int n_units = kb_base + (crank < kb_rem ? 1 : 0);
  const int GL = (C::GROUPS + S - 1) / S;  // most groups any CTA of the cluster owns

  if (threadIdx.x == 0) {
    stamp(a, 7);
    b2::tma_prefetch_desc(&tmP);
    b2::tma_prefetch_desc(&tmQ);
    for (int s = 0; s < STAGES; ++s) {
      b2::mbar_init(bar_full + s * 8, 1);
      b2::mbar_init(bar_empty + s * 8, 1);
    }
    b2::mbar_init(bar_tfull, 1);
    *abort_flag = 0;
    b2::mbar_fence_init();
  }
  if (warp == 1) {
    b2::tmem_alloc(b2::smem_u32(tmem_slot), C::TMEM_COLS);
    b2::tmem_relinquish();
  }
  b2::tc_fence_before();
  __syncthreads();
  b2::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0 && !is_push(EPI)) b2::pdl_launch_dependents();  // fused row-parallel calls: later, see fused_tail
  if (threadIdx.x == 0) stamp(a, 0);
  unsigned int parity = 0;
  // fused qkv heads: rotary factors and cache slots of the first rows this warp will finish, fetched while the
  // mainloop runs (the epilogue warps have nothing else to do then), so that the launch does not end on a chain of
  // dependent global loads
  constexpr int PRE_ROWS = 8;
  float pre_cs[PRE_ROWS][4];
  int pre_slot[PRE_ROWS];

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int pre = n_units < STAGES ? n_units : STAGES;
      for (int i = 0; i < pre; ++i) {  // weights do not depend on earlier kernels
        const uint32_t fb = bar_full + i * 8;
        b2::mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
        b2::tma_load_2d(smem_base + i * C::STAGE_BYTES, &tmP, fb, (kb0 + i) * BK, tile * BM, b2::kEvictFirst);
      }
      b2::pdl_wait();
      stamp(a, 3);
      for (int i = 0; i < pre; ++i)
        b2::tma_load_2d(smem_base + i * C::STAGE_BYTES + C::P_BYTES, &tmQ, bar_full + i * 8, (kb0 + i) * BK, tok0, b2::kEvictLast);
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int i = pre; i < n_units; ++i) {
        if (!b2::mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_EMPTY)) break;
        const uint32_t fb = bar_full + stage * 8;
        b2::mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
        const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
        b2::tma_load_2d(dst, &tmP, fb, (kb0 + i) * BK, tile * BM, b2::kEvictFirst);
        b2::tma_load_2d(dst + C::P_BYTES, &tmQ, fb, (kb0 + i) * BK, tok0, b2::kEvictLast);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = b2::umma_idesc_bf16(BN);
      b2::pdl_wait();  // the pipeline's time limit must not include the wait for earlier kernels
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < n_units; ++i) {
        if (!b2::mbar_wait(bar_full + stage * 8, phase, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_FULL)) { ok = false; break; }
        if (i == 0) stamp(a, 1);
        b2::tc_fence_after();
        const uint32_t sp = smem_base + stage * C::STAGE_BYTES;
        const uint64_t dp = b2::umma_smem_desc(sp);
        const uint64_t dq = b2::umma_smem_desc(sp + C::P_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) b2::umma_bf16(tmem_base, dp + 2 * k, dq + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        b2::umma_commit(bar_empty + stage * 8);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) b2::umma_commit(bar_tfull);
      stamp(a, 2);
    }
  } else {
    // ---------------- epilogue, first half: hand every group of the accumulator to the CTA that owns it ----------------
    const int q = warp & 3;
    const int f = q * 32 + lane;  // feature row of the tile this thread holds
    b2::pdl_wait();
    if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
    if (EPI == EPI_STORE && a.qkv_fused) {
      const bool rotated = tile < a.nq + a.nkv;
#pragma unroll
      for (int i = 0; i < PRE_ROWS; ++i) {
        const int lt = (warp - 2) + 4 * i;
        const int token = tok0 + (((lt >> 2) * S + crank) << 2) + (lt & 3);
        pre_slot[i] = -1;
        pre_cs[i][0] = pre_cs[i][1] = pre_cs[i][2] = pre_cs[i][3] = 0.f;
        if (token < a.M && (lt >> 2) * S + crank < C::GROUPS) {
          if (a.k_cache != nullptr && tile >= a.nq) pre_slot[i] = __ldg(a.slots + token);
          if (rotated) {
            const float* cs = a.cos_sin + __ldg(a.positions + token) * 128;
            pre_cs[i][0] = __ldg(cs + lane * 2); pre_cs[i][1] = __ldg(cs + lane * 2 + 1);
            pre_cs[i][2] = __ldg(cs + 64 + lane * 2); pre_cs[i][3] = __ldg(cs + 64 + lane * 2 + 1);
          }
        }
      }
    }
    if (b2::mbar_wait(bar_tfull, 0, abort_flag, PIPE_LIMIT_NS, B2_WAIT_TMEM_FULL)) {
      b2::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t red_local = b2::smem_u32(red_buf);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        b2::tmem_ld_32x32(taddr + c * 32, r);
        b2::tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int g = c * 8 + j, owner = g % S, gl = g / S;
          const uint32_t local = red_local + ((crank * GL + gl) * BM + f) * 16;
          b2::st_cluster_v4(b2::map_to_cta(local, owner), __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
      }
    }
  }

  // ---- every thread of the cluster meets: all parts have been delivered ----
  __syncwarp();
  b2::cluster_arrive();
  b2::cluster_wait();

  if (warp >= 2 && !*abort_flag) {
    // ---------------- epilogue, second half: sum the S parts of the owned groups, stage, store whole token rows ----------------
    const int q = warp & 3;
    const int f = q * 32 + lane;
    const int feature = tile * BM + f;
    float bias = 0.f;
    if (a.bias != nullptr && feature < a.N) bias = __uint_as_float(static_cast<uint32_t>(a.bias[feature]) << 16);
    uint16_t* out16 = reinterpret_cast<uint16_t*>(out_buf);
    int owned = 0;
    for (int gl = 0; gl < GL; ++gl) {
      const int g = gl * S + crank;
      if (g >= C::GROUPS) break;
      float4 sum = make_float4(bias, bias, bias, bias);
      for (int src = 0; src < S; ++src) {
        const float4 t = *reinterpret_cast<const float4*>(red_buf + ((src * GL + gl) * BM + f) * 16);
        sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
      }
      const uint32_t lo = b2::pack_bf16(sum.x, sum.y), hi = b2::pack_bf16(sum.z, sum.w);
      out16[(gl * 4 + 0) * BM + f] = static_cast<uint16_t>(lo & 0xFFFF);
      out16[(gl * 4 + 1) * BM + f] = static_cast<uint16_t>(lo >> 16);
      out16[(gl * 4 + 2) * BM + f] = static_cast<uint16_t>(hi & 0xFFFF);
      out16[(gl * 4 + 3) * BM + f] = static_cast<uint16_t>(hi >> 16);
      owned = gl + 1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
    if (EPI == EPI_STORE && a.qkv_fused) {
      // The tile is one attention head (128 features) and out_buf holds whole head rows of the tokens this CTA
      // owns: finish the head here.  One warp per token row; lane l holds dims (2l, 2l+1) of both halves.
      // q and k heads: RMSNorm over the head (nanovllm/models/qwen3.py:82-84), neox RoPE
      // (nanovllm/layers/rotary_embedding.py:6-14); k and v heads also go to the paged cache
      // (nanovllm/layers/attention.py:21-30).  Same arithmetic and roundings as qk_norm_rope_store_kernel.
      const bool is_q = tile < a.nq, is_k = !is_q && tile < a.nq + a.nkv;
      const int kvh = is_k ? tile - a.nq : tile - a.nq - a.nkv;
      const uint16_t* nw = (is_q || is_k) ? (is_q ? a.q_norm_w : a.k_norm_w) : nullptr;
      float nw1[2] = {1.f, 1.f}, nw2[2] = {1.f, 1.f};
      if (nw != nullptr) {
        nw1[0] = __uint_as_float(static_cast<uint32_t>(nw[lane * 2]) << 16); nw1[1] = __uint_as_float(static_cast<uint32_t>(nw[lane * 2 + 1]) << 16);
        nw2[0] = __uint_as_float(static_cast<uint32_t>(nw[64 + lane * 2]) << 16); nw2[1] = __uint_as_float(static_cast<uint32_t>(nw[64 + lane * 2 + 1]) << 16);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {  // at most 64 owned rows, 4 warps
        const int lt = (warp - 2) + 4 * i;
        if (lt >= owned * 4) break;
        const int token = tok0 + (((lt >> 2) * S + crank) << 2) + (lt & 3);
        if (token >= a.M) continue;
        const uint16_t* row = out16 + lt * BM;
        uint32_t lo = *reinterpret_cast<const uint32_t*>(row + lane * 2);
        uint32_t hi = *reinterpret_cast<const uint32_t*>(row + 64 + lane * 2);
        int slot;
        float cs4[4];
        if (i < PRE_ROWS) {
          slot = pre_slot[i];
          cs4[0] = pre_cs[i][0]; cs4[1] = pre_cs[i][1]; cs4[2] = pre_cs[i][2]; cs4[3] = pre_cs[i][3];
        } else {  // more rows than were prefetched (no K split: the CTA owns all 64 tokens)
          slot = (a.k_cache != nullptr && !is_q) ? __ldg(a.slots + token) : -1;
          const float* cs = a.cos_sin + __ldg(a.positions + token) * 128;
          cs4[0] = __ldg(cs + lane * 2); cs4[1] = __ldg(cs + lane * 2 + 1);
          cs4[2] = __ldg(cs + 64 + lane * 2); cs4[3] = __ldg(cs + 64 + lane * 2 + 1);
        }
        if (is_q || is_k) {
          float x1[2] = {b2::bf16_lo(lo), b2::bf16_hi(lo)}, x2[2] = {b2::bf16_lo(hi), b2::bf16_hi(hi)};
          if (nw != nullptr) {
            float ss = x1[0] * x1[0] + x2[0] * x2[0] + x1[1] * x1[1] + x2[1] * x2[1];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rstd = rsqrtf(ss / 128.0f + a.qk_eps);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              x1[e] = b2::bf16_round(b2::bf16_round(x1[e] * rstd) * nw1[e]);
              x2[e] = b2::bf16_round(b2::bf16_round(x2[e] * rstd) * nw2[e]);
            }
          }
          float y1[2], y2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            y1[e] = __fsub_rn(__fmul_rn(x1[e], cs4[e]), __fmul_rn(x2[e], cs4[2 + e]));
            y2[e] = __fadd_rn(__fmul_rn(x2[e], cs4[e]), __fmul_rn(x1[e], cs4[2 + e]));
          }
          lo = b2::pack_bf16(y1[0], y1[1]);
          hi = b2::pack_bf16(y2[0], y2[1]);
        }
        uint16_t* dst = a.C + token * a.ldc + tile * BM;
        *reinterpret_cast<uint32_t*>(dst + lane * 2) = lo;
        *reinterpret_cast<uint32_t*>(dst + 64 + lane * 2) = hi;
        if (slot >= 0) {
          uint16_t* cache = (is_k ? a.k_cache : a.v_cache) + (static_cast<int64_t>(slot) * a.nkv + kvh) * 128;
          *reinterpret_cast<uint32_t*>(cache + lane * 2) = lo;
          *reinterpret_cast<uint32_t*>(cache + 64 + lane * 2) = hi;
        }
      }
    } else {
    // rows of out_buf: local token index lt = gl * 4 + j  <->  token (gl * S + crank) * 4 + j; 16 pieces of 16 bytes per row
    const int et = threadIdx.x - 64;
    for (int idx = et; idx < owned * 4 * 16; idx += 128) {
      const int lt = idx >> 4, piece = idx & 15;
      const int token = tok0 + (((lt >> 2) * S + crank) << 2) + (lt & 3);
      const int feat = tile * BM + piece * 8;
      if (token < a.M && feat < a.N) {
        uint4 w = *reinterpret_cast<const uint4*>(out_buf + lt * (BM * 2) + piece * 16);
        if (EPI == EPI_STORE) {
          if (a.silu_pairs) *reinterpret_cast<uint2*>(a.C + token * a.ldc + (feat >> 1)) = silu_mul_pairs(w);
          else *reinterpret_cast<uint4*>(a.C + token * a.ldc + feat) = w;
        } else if (EPI == EPI_PUSH3) {
          w.x = b2::scrub_sentinel(w.x); w.y = b2::scrub_sentinel(w.y);
          w.z = b2::scrub_sentinel(w.z); w.w = b2::scrub_sentinel(w.w);
          int lrow;
          const int owner = owner3_of(token, a.world, lrow);
          *reinterpret_cast<uint4*>(a.inbox[owner] + parity * a.parity_stride + a.rank * a.slot_stride +
                                    (static_cast<size_t>(lrow) * a.N + feat) * 2) = w;
        } else {
          w.x = b2::scrub_sentinel(w.x); w.y = b2::scrub_sentinel(w.y);
          w.z = b2::scrub_sentinel(w.z); w.w = b2::scrub_sentinel(w.w);
          const size_t off = parity * a.parity_stride + a.rank * a.slot_stride + (static_cast<size_t>(token) * a.N + feat) * 2;
#pragma unroll
          for (int r = 0; r < B2_MAX_WORLD; ++r)
            if (r < a.world) *reinterpret_cast<uint4*>(a.inbox[r] + off) = w;
        }
      }
    }
    }
    if (warp == 2 && lane == 0) stamp(a, 4);
  }

  // ---- all roles meet; tensor memory goes back ------------------------------
  b2::pdl_wait();
  if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
  __syncwarp();
  b2::tc_fence_before();
  __syncthreads();
  b2::tc_fence_after();
  const int aborted = *abort_flag;
  if (aborted) {
    for (int i = 0; i < 100; ++i) __nanosleep(2000);
    if (threadIdx.x == 0) b2::report_timeout(a.status, aborted);
  }
  if (warp == 1) b2::tmem_dealloc(tmem_base, C::TMEM_COLS);
  fused_tail<EPI>(a, parity, red, abort_flag, aborted);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) and occupancy answers belong to
// a device, not to the process: one flag per device ordinal, set under a lock.
constexpr int MAX_DEVICES = 64;
std::mutex g_config_mutex;
struct PerDeviceOnce {
  bool done[MAX_DEVICES] = {};
  // runs `configure` the first time it is asked for the current device; returns B2_OK or its error
  template <class F>
  int ensure(F&& configure) {
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return b2::set_error(B2_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_config_mutex);
    if (done[dev]) return B2_OK;
    const int rc = configure();
    if (rc == B2_OK) done[dev] = true;
    return rc;
  }
};

// ---------------------------------------------------------------------------
// Many tokens (prefill, large two-shot calls): CTA pairs.  Two CTAs of a cluster (ranks 0 and 1) run one
// tcgen05.mma.cta_group::2 of 256 token rows x BN features: each CTA stages its own 128 rows of the activations
// and its own half (BN / 2 rows) of the weight tile, the tensor cores of both SMs read the two halves of the
// weight tile from both shared memories, and each CTA's tensor memory receives its 128 rows of the result.
// Per SM and K block that is 16 KB + BN * 64 B of operands from L2 instead of 16 KB + BN * 128 B: the token-row
// GEMM is limited by exactly that traffic.
//   - every CTA:  TMA producer (warp 0) fills its own stages; completion bytes of both CTAs are counted on the
//                 even CTA's "full" barrier; 4 epilogue warps drain the CTA's own tensor memory.
//   - even CTA:   its MMA thread (warp 1) waits on "full", issues the MMAs for the pair, and signals "stage
//                 free" and "accumulator ready" to both CTAs with multicast commits.
//   - odd CTA:    its epilogue warps report "accumulator drained" to the even CTA's barrier.
// Whole 256 x BN tiles are dealt round-robin to the pairs (no K split).  The default for at least 512 tokens.
// ---------------------------------------------------------------------------
template <int BN>
struct CfgPair {
  static constexpr uint32_t P_BYTES = BM * BK * 2;            // this CTA's 128 token rows
  static constexpr uint32_t Q_BYTES = (BN / 2) * BK * 2;      // this CTA's half of the weight tile
  static constexpr uint32_t STAGE_BYTES = P_BYTES + Q_BYTES;
  static constexpr int ACC = 512 / BN;                        // accumulators in tensor memory (512 columns in all)
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr int STAGES_RAW = (232448 - 1024 - 256 - 4 * STAGING_BYTES_PER_WARP) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + 4 * STAGING_BYTES_PER_WARP;
  static_assert(BN == 128 || BN == 256, "pair tiles are 256 x 128 or 256 x 256");
  static_assert(2 * STAGES + 2 * ACC <= 30, "barrier area is 256 bytes");
};

template <int BN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, const GemmArgs a) {
  using C = CfgPair<BN>;
  constexpr int STAGES = C::STAGES, ACC = C::ACC;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = b2::smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  const uint32_t bar_full = b2::smem_u32(bars);             // used in the even CTA: bytes of both CTAs' loads
  const uint32_t bar_empty = bar_full + STAGES * 8;         // in each CTA: its stage may be refilled
  const uint32_t bar_tfull = bar_empty + STAGES * 8;        // in each CTA: accumulator complete
  const uint32_t bar_tempty = bar_tfull + ACC * 8;          // used in the even CTA: both CTAs' epilogues have drained it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float red[NUM_THREADS / 32];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = b2::cluster_ctarank();                // 0 = even CTA (issues the MMAs), 1 = odd CTA
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int KB = a.kblocks;
  const int tiles2 = a.tilesP * a.tilesQ;                   // tilesP counts 256-row tiles here
  const int my_tiles = pair < tiles2 ? (tiles2 - pair + pairs - 1) / pairs : 0;
  const int n_units = my_tiles * KB;

  if (threadIdx.x == 0) {
    stamp(a, 7);
    b2::tma_prefetch_desc(&tmP);
    b2::tma_prefetch_desc(&tmQ);
    for (int s = 0; s < STAGES; ++s) {
      b2::mbar_init(bar_full + s * 8, 1);
      b2::mbar_init(bar_empty + s * 8, 1);
    }
    for (int i = 0; i < ACC; ++i) {
      b2::mbar_init(bar_tfull + i * 8, 1);
      b2::mbar_init(bar_tempty + i * 8, 8);  // 4 epilogue warps of each of the 2 CTAs
    }
    *abort_flag = 0;
    b2::mbar_fence_init();
  }
  if (warp == 1) {
    b2::tmem_alloc_pair(b2::smem_u32(tmem_slot), C::TMEM_COLS);
    b2::tmem_relinquish_pair();
  }
  b2::tc_fence_before();
  __syncthreads();
  // the other CTA's barriers must exist before anything is counted on them
  b2::cluster_arrive();
  b2::cluster_wait();
  b2::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0 && !is_push(EPI)) b2::pdl_launch_dependents();  // fused row-parallel calls: later, see fused_tail
  if (threadIdx.x == 0) stamp(a, 0);
  unsigned int parity = 0;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      const uint32_t full0 = b2::map_to_cta(bar_full, 0);   // the even CTA's "full" barriers, as a cluster address
      const int pre = n_units < STAGES ? n_units : STAGES;
      int t = pair, kb = 0;                                 // tile and K block of the unit being loaded
      // weights of the first stages depend on no earlier kernel
      for (int i = 0; i < pre; ++i) {
        if (cr == 0) b2::mbar_arrive_expect_tx(bar_full + i * 8, 2 * C::STAGE_BYTES);
        const int tq = t % a.tilesQ;
        b2::tma_load_2d_pair(smem_base + i * C::STAGE_BYTES + C::P_BYTES, &tmQ, full0 + i * 8, kb * BK,
                             tq * BN + static_cast<int>(cr) * (BN / 2), b2::kEvictNormal);
        if (++kb == KB) { kb = 0; t += pairs; }
      }
      b2::pdl_wait();
      stamp(a, 3);
      t = pair;
      kb = 0;
      for (int i = 0; i < pre; ++i) {
        const int tp = t / a.tilesQ;
        b2::tma_load_2d_pair(smem_base + i * C::STAGE_BYTES, &tmP, full0 + i * 8, kb * BK, (tp * 2 + static_cast<int>(cr)) * BM,
                             b2::kEvictNormal);
        if (++kb == KB) { kb = 0; t += pairs; }
      }
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int i = pre; i < n_units; ++i) {
        if (!b2::mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_EMPTY)) break;
        if (cr == 0) b2::mbar_arrive_expect_tx(bar_full + stage * 8, 2 * C::STAGE_BYTES);
        const int tp = t / a.tilesQ, tq = t - tp * a.tilesQ;
        const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
        b2::tma_load_2d_pair(dst, &tmP, full0 + stage * 8, kb * BK, (tp * 2 + static_cast<int>(cr)) * BM, b2::kEvictNormal);
        b2::tma_load_2d_pair(dst + C::P_BYTES, &tmQ, full0 + stage * 8, kb * BK, tq * BN + static_cast<int>(cr) * (BN / 2),
                             b2::kEvictNormal);
        if (++kb == KB) { kb = 0; t += pairs; }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && cr == 0) {
      constexpr uint32_t idesc = b2::umma_idesc_bf16_pair(BN);
      b2::pdl_wait();  // the pipeline's time limit must not include the wait for earlier kernels
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int j = 0; ok && j < my_tiles; ++j) {
        const int acc = j % ACC;
        const uint32_t use = static_cast<uint32_t>(j / ACC);
        if (!b2::mbar_wait(bar_tempty + acc * 8, (use & 1) ^ 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_TMEM_EMPTY)) break;
        b2::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!b2::mbar_wait(bar_full + stage * 8, phase, abort_flag, PIPE_LIMIT_NS, B2_WAIT_SMEM_FULL)) { ok = false; break; }
          if (j == 0 && kb == 0) stamp(a, 1);
          b2::tc_fence_after();
          const uint32_t sp = smem_base + stage * C::STAGE_BYTES;
          const uint64_t dp = b2::umma_smem_desc(sp);
          const uint64_t dq = b2::umma_smem_desc(sp + C::P_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) b2::umma_bf16_pair(d_tmem, dp + 2 * k, dq + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          b2::umma_commit_pair(bar_empty + stage * 8, 3);   // both CTAs may refill this stage
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        b2::umma_commit_pair(bar_tfull + acc * 8, 3);       // both CTAs may drain their half of the accumulator
      }
      stamp(a, 2);
    }
  } else {
    // ---------------- epilogue warps (both CTAs) ----------------
    const int q = warp & 3;
    unsigned char* wbuf = smem + STAGES * C::STAGE_BYTES + 256 + q * STAGING_BYTES_PER_WARP;
    const uint32_t tempty0 = b2::map_to_cta(bar_tempty, 0);
    b2::pdl_wait();
    if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
    for (int j = 0; j < my_tiles; ++j) {
      const int t = pair + j * pairs;
      const int acc = j % ACC;
      const uint32_t use = static_cast<uint32_t>(j / ACC);
      if (!b2::mbar_wait(bar_tfull + acc * 8, use & 1, abort_flag, PIPE_LIMIT_NS, B2_WAIT_TMEM_FULL)) break;
      b2::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int tp = t / a.tilesQ, tq = t - tp * a.tilesQ;
      const int p_row = (tp * 2 + static_cast<int>(cr)) * BM + q * 32 + lane;  // token row of this lane
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        b2::tmem_ld_32x32(taddr + c * 32, r);
        b2::tc_wait_ld();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        emit_chunk<BN, false, EPI>(a, v, p_row, tq * BN, c, lane, parity, wbuf, 0u, nullptr);
      }
      b2::tc_fence_before();
      __syncwarp();
      if (lane == 0) b2::mbar_arrive_cluster(tempty0 + acc * 8);
    }
    if (warp == 2 && lane == 0) stamp(a, 4);
  }

  // ---- all roles of both CTAs meet; tensor memory goes back ------------------
  b2::pdl_wait();
  if (is_push(EPI)) parity = *reinterpret_cast<volatile unsigned int*>(&a.dstate->rowpar_seq) & 1u;
  __syncwarp();
  b2::tc_fence_before();
  __syncthreads();
  const int aborted = *abort_flag;
  if (aborted) {
    // let bulk copies that may still be in flight (this CTA's and the other's) land before anyone leaves
    for (int i = 0; i < 100; ++i) __nanosleep(2000);
    if (threadIdx.x == 0) b2::report_timeout(a.status, aborted);
  }
  // neither CTA may free the pair's tensor memory or leave while the other still signals its barriers
  b2::cluster_arrive();
  b2::cluster_wait();
  b2::tc_fence_after();
  if (warp == 1) b2::tmem_dealloc_pair(tmem_base, C::TMEM_COLS);

  fused_tail<EPI>(a, parity, red, abort_flag, aborted);
}

template <int BN, bool SWAP, int EPI>
int launch_inst(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmArgs& args, int grid, cudaStream_t stream) {
  static PerDeviceOnce configured;
  constexpr uint32_t smem_bytes = SWAP ? Cfg<BN>::SMEM_BYTES : Cfg<BN>::SMEM_BYTES_ROWS;
  static_assert(smem_bytes <= 232448, "more shared memory than an SM has");
  const int crc = configured.ensure([&]() -> int {
    B2_CUDA(cudaFuncSetAttribute(gemm_kernel<BN, SWAP, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    return B2_OK;
  });
  if (crc != B2_OK) return crc;
  B2_CUDA(b2_launch(gemm_kernel<BN, SWAP, EPI>, dim3(grid), dim3(NUM_THREADS), smem_bytes, stream, tmP, tmQ, args));
  return B2_OK;
}

template <int BN, int EPI>
int configure_cluster_kernel() {
  static PerDeviceOnce configured;
  return configured.ensure([&]() -> int {
    B2_CUDA(cudaFuncSetAttribute(gemm_cluster_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgCluster<BN>::SMEM_BYTES));
    return B2_OK;
  });
}

template <int BN, int EPI>
int launch_cluster_inst(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmArgs& args, int tiles, int S, cudaStream_t stream) {
  const int crc = configure_cluster_kernel<BN, EPI>();
  if (crc != B2_OK) return crc;
  B2_CUDA(b2_launch_cluster(gemm_cluster_kernel<BN, EPI>, dim3(tiles * S), dim3(NUM_THREADS), CfgCluster<BN>::SMEM_BYTES, stream,
                            static_cast<unsigned>(S), tmP, tmQ, args));
  return B2_OK;
}

template <int BN, int EPI>
int launch_pair_inst(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmArgs& args, int grid, cudaStream_t stream) {
  static PerDeviceOnce configured;
  const int crc = configured.ensure([&]() -> int {
    B2_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgPair<BN>::SMEM_BYTES));
    return B2_OK;
  });
  if (crc != B2_OK) return crc;
  B2_CUDA(b2_launch_cluster(gemm_pair_kernel<BN, EPI>, dim3(grid), dim3(NUM_THREADS), CfgPair<BN>::SMEM_BYTES, stream, 2u, tmP, tmQ, args));
  return B2_OK;
}

// The CTA-pair kernel serves many-token problems (at least 512 tokens, tiles of 128 or 256 features); B2_PAIR=0 in
// the environment sends them to the stream-K kernel instead (for comparison).
bool pair_path_enabled() {
  static const bool on = [] {
    const char* e = getenv("B2_PAIR");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// How many clusters of S CTAs of the cluster kernel can be resident at once (cached per device, BN and S).
template <int BN, int EPI>
int max_resident_clusters(int S) {
  static int cache[MAX_DEVICES][9];
  static bool cache_init = false;
  if (S < 1 || S > 8) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  {
    std::lock_guard<std::mutex> lock(g_config_mutex);
    if (!cache_init) {
      for (auto& row : cache)
        for (int& v : row) v = -1;
      cache_init = true;
    }
    if (cache[dev][S] >= 0) return cache[dev][S];
  }
  if (configure_cluster_kernel<BN, EPI>() != B2_OK) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S * 64);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = CfgCluster<BN>::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_cluster_kernel<BN, EPI>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  std::lock_guard<std::mutex> lock(g_config_mutex);
  cache[dev][S] = n;
  return n;
}

thread_local int g_last_gemm_path = 0;  // 0 = stream-K kernel, 1 = cluster kernel, 2 = CTA-pair kernel (set by launch_gemm)

// What launch_gemm decides for one problem, as data (the CPU tests read it through b2_plan_gemm).
struct GemmPlan {
  int swap;           // 1 = feature-lane layout (weights on the 128-row side)
  int bn;             // rows of the Q tile
  int tilesP, tilesQ, kblocks;
  int gemm_ctas;      // CTAs that share the GEMM units
  int round_robin;    // stream-K kernel: whole tiles dealt round-robin
  int grid;           // CTAs launched
  int cluster_split;  // > 0: cluster kernel with this K split; 0: stream-K kernel
};

// Picks the K split S of the cluster kernel for `tiles` output tiles of `kblocks` K blocks: the largest S that
// keeps every cluster resident in one wave and leaves each CTA at least two K blocks.  0 = use the stream-K kernel.
// resident(bn, S) = how many clusters of S CTAs fit on the device at once.
template <class Resident>
int pick_cluster_split(int bn, int tiles, int kblocks, int num_sms, Resident&& resident) {
  if (tiles > num_sms) return 0;
  for (int S = 8; S >= 1; --S) {
    if (S > 1 && kblocks < 2 * S) continue;
    if (tiles * S > num_sms) continue;
    if (resident(bn, S) >= tiles) return S;
  }
  return 0;
}

// Pure host arithmetic: no CUDA call besides what `resident` makes.
constexpr int PLAN_WHOLE_TILES = 1;  // planner option bit

// Planner option PLAN_WHOLE_TILES (b2_ctx_set_option B2_OPT_WHOLE_TILES): a token-row problem whose tiles fit the device
// in one wave at some tile width runs one whole tile per CTA instead of a stream-K split, whose fp32 combine in L2 costs
// more than the idle SMs when the GEMM itself lasts a few microseconds (128-1024 tokens of a fused row-parallel call).

template <class Resident>
int plan_gemm(int epi, int M, int N, int K, int num_sms, int min_grid, int reducers, int64_t tile_cap, bool clusters_on,
              Resident&& resident, GemmPlan& p, int options = 0) {
  if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return B2_ERR_ARG;
  p.swap = (epi != EPI_PUSH2) && M <= (epi == EPI_PUSH3 ? 64 : 256);  // the owner form sends whole row segments: token rows above the decode sizes
  if (p.swap) p.bn = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  else p.bn = (N >= 256) ? 256 : (N > 64 ? 128 : 64);
  bool one_tile_per_cta = false;
  // (a whole tile per CTA means the CTA walks the whole K range alone: worth it only while that range is short)
  if (!p.swap && (options & PLAN_WHOLE_TILES) && (K + BK - 1) / BK <= 96) {
    const int sms = epi == EPI_PUSH2 ? std::max(1, num_sms - reducers) : num_sms;
    for (int bn = 64; bn <= p.bn; bn *= 2) {  // the narrowest tile that still fits one wave gives the most parallelism
      const int64_t t = static_cast<int64_t>((M + BM - 1) / BM) * ((N + bn - 1) / bn);
      if (t <= sms) {
        p.bn = bn;
        one_tile_per_cta = true;
        break;
      }
    }
  }
  const int rowsP = p.swap ? N : M, rowsQ = p.swap ? M : N;
  p.tilesP = (rowsP + BM - 1) / BM;
  p.tilesQ = (rowsQ + p.bn - 1) / p.bn;
  p.kblocks = (K + BK - 1) / BK;
  const int64_t tiles = static_cast<int64_t>(p.tilesP) * p.tilesQ;
  if (tiles > tile_cap) return B2_ERR_SHAPE;
  const int64_t U = tiles * p.kblocks;
  if (U > (1ll << 30)) return B2_ERR_SHAPE;
  // every CTA should stream at least ~8 K blocks, or splitting costs more than it saves
  int64_t g = std::max<int64_t>(1, U / 8);
  const int sms_for_gemm = epi == EPI_PUSH2 ? std::max(1, num_sms - reducers) : num_sms;
  g = std::min<int64_t>(g, sms_for_gemm);
  g = std::min<int64_t>(g, U);
  p.gemm_ctas = static_cast<int>(g);
  p.round_robin = (!p.swap && tiles >= 4 * g) ? 1 : 0;
  if (one_tile_per_cta) {
    p.gemm_ctas = static_cast<int>(tiles);
    p.round_robin = 1;
  }
  p.grid = (epi == EPI_PUSH2 || epi == EPI_PUSH3) ? num_sms : std::max(p.gemm_ctas, std::min(min_grid, num_sms));
  p.cluster_split = 0;
  if ((epi == EPI_STORE || epi == EPI_PUSH || epi == EPI_PUSH3) && clusters_on && p.swap && p.tilesQ == 1 && p.bn <= 64) {  // up to 64 tokens: the decode sizes
    p.cluster_split = pick_cluster_split(p.bn, p.tilesP, p.kblocks, num_sms, resident);
    if (p.cluster_split > 0) {
      p.gemm_ctas = p.tilesP * p.cluster_split;
      p.grid = p.gemm_ctas;
    }
  } else if ((epi == EPI_STORE || epi == EPI_PUSH) && clusters_on && p.swap && M > 64) {
    // 65..256 tokens: the cluster kernel over 64-token tiles when all (feature tile, token tile) pairs fit one wave -
    // no fp32 combine through L2, which costs these few-microsecond problems more than the GEMM itself
    const int tq64 = (M + 63) / 64;
    const int64_t pairs = static_cast<int64_t>(p.tilesP) * tq64;
    int split = 0;
    if (pairs <= num_sms) split = pick_cluster_split(64, static_cast<int>(pairs), p.kblocks, num_sms, resident);
    // a plain GEMM's CTAs wait for nobody, so its tiles need not be resident together: up to 4 waves of unsplit tiles
    else if (epi == EPI_STORE && pairs <= 4 * static_cast<int64_t>(num_sms) && p.kblocks <= 48 && resident(64, 1) > 0) split = 1;
    {
      // (only while a CTA's share of K stays short: with a long K range and no room to split it, stream-K over all SMs wins)
      if (split > 0 && (p.kblocks + split - 1) / split <= 32) {
        p.bn = 64;
        p.tilesQ = tq64;
        p.cluster_split = split;
        p.gemm_ctas = static_cast<int>(pairs) * split;
        p.grid = p.gemm_ctas;
      }
    }
  }
  return B2_OK;
}

template <int EPI>
int launch_gemm(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K, GemmArgs& args,
                int min_grid, cudaStream_t stream) {
  const int reducers = 0;  // no CTAs are set aside for the reduce phase: every CTA reduces after its GEMM work
  GemmPlan plan;
  const int prc = plan_gemm(EPI, M, N, K, ctx->num_sms, min_grid, reducers, ctx->tile_counter_cap, true,
                            [](int bn, int S) {
                              if constexpr (EPI == EPI_PUSH2 || EPI == EPI_SAMPLE) return 0;
                              else return bn == 32 ? max_resident_clusters<32, EPI>(S) : max_resident_clusters<64, EPI>(S);
                            },
                            plan, (ctx->whole_tiles && (EPI == EPI_PUSH2 || EPI == EPI_PUSH3)) ? PLAN_WHOLE_TILES : 0);
  if (prc != B2_OK) return prc;
  const bool swap = plan.swap != 0;
  const int bn = plan.bn;
  const int rowsP = swap ? N : M, rowsQ = swap ? M : N;
  args.tilesP = plan.tilesP;
  args.tilesQ = plan.tilesQ;
  args.kblocks = plan.kblocks;
  args.M = M;
  args.N = N;
  args.ws = ctx->splitk_ws;
  args.counters = ctx->tile_counters;
  args.status = ctx->status_dev;
  args.trace = ctx->trace_on ? ctx->trace : nullptr;
  args.gemm_ctas = plan.gemm_ctas;
  args.round_robin = plan.round_robin;
  const int grid = plan.grid;

  CUtensorMap tmP, tmQ;
  const void* pP = swap ? W : A;
  const void* pQ = swap ? A : W;
  const int64_t ldP = swap ? ldw : lda, ldQ = swap ? lda : ldw;
  int rc = b2::encode_tmap_2d(&tmP, pP, K, rowsP, ldP, BK, BM);
  if (rc != B2_OK) return rc;
  rc = b2::encode_tmap_2d(&tmQ, pQ, K, rowsQ, ldQ, BK, bn);
  if (rc != B2_OK) return rc;

  g_last_gemm_path = 0;
  if constexpr (EPI == EPI_STORE || EPI == EPI_PUSH2) {
    // CTA pairs (tcgen05.mma.cta_group::2) for many-token problems: 1.1-1.2x the stream-K kernel from 512 tokens on
    if (pair_path_enabled() && !swap && bn >= 128 && M >= 512 && ctx->num_sms >= 2) {
      CUtensorMap tmQh;
      rc = b2::encode_tmap_2d(&tmQh, pQ, K, rowsQ, ldQ, BK, bn / 2);
      if (rc != B2_OK) return rc;
      args.tilesP = (M + 2 * BM - 1) / (2 * BM);
      args.gemm_ctas = ctx->num_sms & ~1;
      args.round_robin = 1;
      g_last_gemm_path = 2;
      if (bn == 128) return launch_pair_inst<128, EPI>(tmP, tmQh, args, args.gemm_ctas, stream);
      return launch_pair_inst<256, EPI>(tmP, tmQh, args, args.gemm_ctas, stream);
    }
  }
  if constexpr (EPI == EPI_STORE || EPI == EPI_PUSH || EPI == EPI_PUSH3) {
    if (plan.cluster_split > 0) {
      g_last_gemm_path = 1;
      if (bn == 32) return launch_cluster_inst<32, EPI>(tmP, tmQ, args, args.tilesP * args.tilesQ, plan.cluster_split, stream);
      return launch_cluster_inst<64, EPI>(tmP, tmQ, args, args.tilesP * args.tilesQ, plan.cluster_split, stream);
    }
  }
  if constexpr (EPI == EPI_PUSH3) {
    if (swap) {  // at most 64 tokens in this layout
      if (bn == 32) return launch_inst<32, true, EPI>(tmP, tmQ, args, grid, stream);
      return launch_inst<64, true, EPI>(tmP, tmQ, args, grid, stream);
    }
  } else if constexpr (EPI != EPI_PUSH2) {
    if (swap) {
      switch (bn) {
        case 32: return launch_inst<32, true, EPI>(tmP, tmQ, args, grid, stream);
        case 64: return launch_inst<64, true, EPI>(tmP, tmQ, args, grid, stream);
        case 128: return launch_inst<128, true, EPI>(tmP, tmQ, args, grid, stream);
        default: return launch_inst<256, true, EPI>(tmP, tmQ, args, grid, stream);
      }
    }
  }
  if constexpr (EPI == EPI_SAMPLE) {
    return B2_ERR_SHAPE;  // the fused sampler exists in the feature-lane layout only (at most 256 token rows)
  } else {
    switch (bn) {
      case 64: return launch_inst<64, false, EPI>(tmP, tmQ, args, grid, stream);
      case 128: return launch_inst<128, false, EPI>(tmP, tmQ, args, grid, stream);
      default: return launch_inst<256, false, EPI>(tmP, tmQ, args, grid, stream);
    }
  }
}

int check_operands(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K) {
  if (M < 0 || N <= 0 || K <= 0) return B2_ERR_ARG;
  if (!A || !W || !aligned16(A) || !aligned16(W)) return B2_ERR_ARG;
  if (K % 8 != 0 || N % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K) return B2_ERR_ARG;
  return B2_OK;
}

// rows of h picked by index into a contiguous staging buffer (the prefill
// "last token of every sequence" selection)
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint16_t* __restrict__ h, int64_t ldh,
                                                          const int32_t* __restrict__ idx, int B, int H,
                                                          uint16_t* __restrict__ out) {
  b2::pdl_launch_dependents();
  b2::pdl_wait();
  const int vpr = H >> 3;
  const int64_t total = static_cast<int64_t>(B) * vpr;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(i / vpr), v = static_cast<int>(i - static_cast<int64_t>(b) * vpr);
    *reinterpret_cast<uint4*>(out + static_cast<int64_t>(b) * H + v * 8) =
        __ldg(reinterpret_cast<const uint4*>(h + idx[b] * ldh + v * 8));
  }
}

// Completion of the logits gather.  It runs after the GEMM that stored this
// rank's slice into rank 0's buffer (stream order makes those stores visible
// before anything this kernel writes).  Ranks other than 0 publish the call
// number in rank 0's flag word; rank 0 waits until every peer has published it.
__global__ void lm_head_sync_kernel(int rank, int world, unsigned int* flags_rank0, B2DeviceState* dstate, B2Status* status,
                                    uint64_t timeout_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  b2::pdl_wait();
  const unsigned int want = dstate->lmhead_seq + 1;
  if (rank != 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags_rank0 + rank), "r"(want) : "memory");
  } else {
    const uint64_t t0 = b2::globaltimer_ns();
    for (int r = 1; r < world; ++r) {
      for (uint32_t spin = 0;; ++spin) {
        unsigned int got;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(flags_rank0 + r) : "memory");
        if (static_cast<int>(got - want) >= 0) break;
        if ((spin & 0xFF) == 0xFF && b2::time_limit_passed(t0, timeout_ns)) {
          b2::report_timeout(status, B2_WAIT_LOGITS);
          break;
        }
      }
    }
  }
  dstate->lmhead_seq = want;
}

// Completion of the fused LM-head sampler.  One block.  Every rank hands its best key per row to rank 0
// (its own slot of rank 0's key box, then the call number in rank 0's flag word); rank 0 waits for the
// peers, keeps the largest key of each row and writes the vocabulary ids.  The local table goes back to
// zero and the call counters advance.  The key box alternates between two halves by call number.
__global__ void __launch_bounds__(256) sample_finish_kernel(int rank, int world, int B, int max_seqs, unsigned long long* keys,
                                                            unsigned long long* keybox_rank0, unsigned int* flags_rank0,
                                                            B2DeviceState* dstate, B2Status* status, uint64_t timeout_ns,
                                                            int64_t* tokens_out) {
  b2::pdl_wait();
  const unsigned int want = dstate->lmhead_seq + 1;
  unsigned long long* box = keybox_rank0 + static_cast<size_t>(want & 1u) * world * max_seqs;
  const int t = threadIdx.x;
  unsigned long long best = 0ull;
  if (t < B) {
    best = keys[t];
    keys[t] = 0ull;
  }
  if (world > 1) {
    if (rank != 0) {
      if (t < B) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(box + static_cast<size_t>(rank) * max_seqs + t), "l"(best) : "memory");
      __threadfence_system();
      __syncthreads();
      if (t == 0) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags_rank0 + rank), "r"(want) : "memory");
    } else {
      if (t == 0) {
        const uint64_t t0 = b2::globaltimer_ns();
        for (int r = 1; r < world; ++r) {
          for (uint32_t spin = 0;; ++spin) {
            unsigned int got;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(flags_rank0 + r) : "memory");
            if (static_cast<int>(got - want) >= 0) break;
            if ((spin & 0xFF) == 0xFF && b2::time_limit_passed(t0, timeout_ns)) {
              b2::report_timeout(status, B2_WAIT_LOGITS);
              break;
            }
          }
        }
        __threadfence_system();
      }
      __syncthreads();
      if (t < B) {
        for (int r = 1; r < world; ++r) {
          unsigned long long k;
          asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(k) : "l"(box + static_cast<size_t>(r) * max_seqs + t) : "memory");
          best = k > best ? k : best;
        }
      }
    }
  }
  if (rank == 0 && t < B) tokens_out[t] = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(best));
  __syncthreads();
  if (t == 0) {
    dstate->lmhead_seq = want;
    dstate->sample_seq += 1;
  }
}

}  // namespace

extern "C" {

int b2_lm_head(b2_ctx* ctx, const void* h, int64_t ldh, const int32_t* row_index, const void* W, int64_t ldw, int B, int Vr, int H,
               void** logits_out, void* stream) {
  if (ctx == nullptr || logits_out == nullptr) return B2_ERR_ARG;
  *logits_out = nullptr;
  int rc = check_operands(h, ldh, W, ldw, B, Vr, H);
  if (rc != B2_OK) return rc;
  const int world = ctx->cfg.world, rank = ctx->cfg.rank;
  if (ctx->cfg.vocab <= 0 || ctx->cfg.max_seqs <= 0) return B2_ERR_STATE;
  if (B > ctx->cfg.max_seqs || static_cast<int64_t>(Vr) * world != ctx->cfg.vocab || H > ctx->cfg.hidden) return B2_ERR_SHAPE;
  if (!ctx->peers_ready) return B2_ERR_STATE;
  if (B == 0) return B2_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void* A = h;
  int64_t lda = ldh;
  if (row_index != nullptr) {
    const int64_t work = static_cast<int64_t>(B) * (H / 8);
    const int grid = static_cast<int>(std::min<int64_t>((work + 255) / 256, ctx->num_sms * 4));
    B2_CUDA(b2_launch(gather_rows_kernel, dim3(grid), dim3(256), 0, s, static_cast<const uint16_t*>(h), ldh, row_index, B, H,
                      reinterpret_cast<uint16_t*>(ctx->gather_rows)));
    A = ctx->gather_rows;
    lda = H;
  }
  GemmArgs args{};
  args.C = reinterpret_cast<uint16_t*>(ctx->peer[0] + ctx->off_logits) + static_cast<size_t>(rank) * Vr;
  args.ldc = ctx->cfg.vocab;
  rc = launch_gemm<EPI_STORE>(ctx, A, lda, W, ldw, B, Vr, H, args, 0, s);
  if (rc != B2_OK) return rc;
  if (world > 1) {
    B2_CUDA(b2_launch(lm_head_sync_kernel, dim3(1), dim3(32), 0, s, rank, world, reinterpret_cast<unsigned int*>(ctx->peer[0] + ctx->off_flags),
                      ctx->dstate, ctx->status_dev, static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull));
  }
  if (rank == 0) *logits_out = ctx->symm + ctx->off_logits;
  return B2_OK;
}

int b2_lm_head_sample(b2_ctx* ctx, const void* h, int64_t ldh, const int32_t* row_index, const void* W, int64_t ldw, int B, int Vr,
                      int H, const float* temperatures, uint64_t seed, int64_t* tokens_out, void* stream) {
  if (ctx == nullptr) return B2_ERR_ARG;
  int rc = check_operands(h, ldh, W, ldw, B, Vr, H);
  if (rc != B2_OK) return rc;
  const int world = ctx->cfg.world, rank = ctx->cfg.rank;
  if (rank == 0 && tokens_out == nullptr) return B2_ERR_ARG;
  if (ctx->cfg.vocab <= 0 || ctx->cfg.max_seqs <= 0) return B2_ERR_STATE;
  if (B > ctx->cfg.max_seqs || static_cast<int64_t>(Vr) * world != ctx->cfg.vocab || H > ctx->cfg.hidden) return B2_ERR_SHAPE;
  if (B > 256) return b2::set_error(B2_ERR_SHAPE, "b2_lm_head_sample: %d rows; the fused sampler takes at most 256, use b2_lm_head", B);
  if (!ctx->peers_ready) return B2_ERR_STATE;
  if (B == 0) return B2_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void* A = h;
  int64_t lda = ldh;
  if (row_index != nullptr) {
    const int64_t work = static_cast<int64_t>(B) * (H / 8);
    const int grid = static_cast<int>(std::min<int64_t>((work + 255) / 256, ctx->num_sms * 4));
    B2_CUDA(b2_launch(gather_rows_kernel, dim3(grid), dim3(256), 0, s, static_cast<const uint16_t*>(h), ldh, row_index, B, H,
                      reinterpret_cast<uint16_t*>(ctx->gather_rows)));
    A = ctx->gather_rows;
    lda = H;
  }
  GemmArgs args{};
  args.sample_keys = ctx->sample_keys;
  args.temperatures = temperatures;
  args.seed = seed;
  args.vocab_offset = rank * Vr;
  args.dstate = ctx->dstate;
  rc = launch_gemm<EPI_SAMPLE>(ctx, A, lda, W, ldw, B, Vr, H, args, 0, s);
  if (rc != B2_OK) return rc;
  B2_CUDA(b2_launch(sample_finish_kernel, dim3(1), dim3(256), 0, s, rank, world, B, ctx->cfg.max_seqs, ctx->sample_keys,
                    reinterpret_cast<unsigned long long*>(ctx->peer[0] + ctx->off_keybox),
                    reinterpret_cast<unsigned int*>(ctx->peer[0] + ctx->off_flags), ctx->dstate, ctx->status_dev,
                    static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull, tokens_out));
  return B2_OK;
}

// The fused sampler's noise for one (vocab id, token row, call): host copy of the device arithmetic, for tests.
int b2_sampler_noise_bits(uint64_t seed, uint32_t vocab_id, uint32_t token, uint32_t call, uint32_t* bits) {
  if (bits == nullptr) return B2_ERR_ARG;
  uint32_t r[4] = {vocab_id, token >> 2, call, SAMPLE_TAG};
  philox4x32_10(r, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  *bits = r[token & 3];
  return B2_OK;
}

// Philox4x32-10 itself (counter and key as given), for the known-answer test.
int b2_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
  if (counter == nullptr || key == nullptr || out == nullptr) return B2_ERR_ARG;
  uint32_t r[4] = {counter[0], counter[1], counter[2], counter[3]};
  philox4x32_10(r, key[0], key[1]);
  for (int i = 0; i < 4; ++i) out[i] = r[i];
  return B2_OK;
}

int b2_gemm(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, void* C, int64_t ldc, int M,
            int N, int K, void* stream) {
  if (ctx == nullptr) return B2_ERR_ARG;
  int rc = check_operands(A, lda, W, ldw, M, N, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!C || !aligned16(C) || ldc % 8 != 0 || ldc < N) return B2_ERR_ARG;
  if (bias != nullptr && !aligned16(bias)) return B2_ERR_ARG;
  GemmArgs args{};
  args.C = static_cast<uint16_t*>(C);
  args.ldc = ldc;
  args.bias = static_cast<const uint16_t*>(bias);
  return launch_gemm<EPI_STORE>(ctx, A, lda, W, ldw, M, N, K, args, 0, static_cast<cudaStream_t>(stream));
}

int b2_qkv_fused(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, void* qkv, int64_t ld_qkv, int M,
                 int nq, int nkv, int head_dim, int K, const void* q_norm_w, const void* k_norm_w, float eps, const int64_t* positions,
                 const float* cos_sin, void* k_cache, void* v_cache, const int32_t* slot_mapping, void* stream) {
  if (ctx == nullptr || nq <= 0 || nkv <= 0 || (head_dim != 128 && head_dim != 64)) return B2_ERR_ARG;
  const int N = (nq + 2 * nkv) * head_dim;
  int rc = check_operands(A, lda, W, ldw, M, N, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!qkv || !aligned16(qkv) || ld_qkv % 8 != 0 || ld_qkv < N || !positions || !cos_sin) return B2_ERR_ARG;
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return B2_ERR_ARG;
  if (k_cache != nullptr && (!v_cache || !slot_mapping)) return B2_ERR_ARG;
  if (bias != nullptr && !aligned16(bias)) return B2_ERR_ARG;
  GemmArgs args{};
  args.C = static_cast<uint16_t*>(qkv);
  args.ldc = ld_qkv;
  args.bias = static_cast<const uint16_t*>(bias);
  if (head_dim == 128) {  // one head per 128-feature tile: the cluster kernel can finish the heads itself
    args.qkv_fused = 1;
    args.nq = nq;
    args.nkv = nkv;
    args.positions = positions;
    args.cos_sin = cos_sin;
    args.q_norm_w = static_cast<const uint16_t*>(q_norm_w);
    args.k_norm_w = static_cast<const uint16_t*>(k_norm_w);
    args.qk_eps = eps;
    args.k_cache = static_cast<uint16_t*>(k_cache);
    args.v_cache = static_cast<uint16_t*>(v_cache);
    args.slots = slot_mapping;
  }
  rc = launch_gemm<EPI_STORE>(ctx, A, lda, W, ldw, M, N, K, args, 0, static_cast<cudaStream_t>(stream));
  if (rc != B2_OK) return rc;
  if (args.qkv_fused && g_last_gemm_path == 1) return B2_OK;
  // many tokens (or 64-wide heads): the projection ran on the stream-K kernel; finish the heads in a second launch
  return b2_qk_norm_rope_store(qkv, ld_qkv, M, nq, nkv, head_dim, q_norm_w, k_norm_w, eps, positions, cos_sin, k_cache, v_cache, slot_mapping,
                               stream);
}

int b2_gemm_silu_mul(b2_ctx* ctx, const void* A, int64_t lda, const void* W_pairs, int64_t ldw, void* out, int64_t ldo, int M, int I, int K,
                     void* stream) {
  if (ctx == nullptr) return B2_ERR_ARG;
  if (I <= 0 || I % 8 != 0) return B2_ERR_ARG;
  int rc = check_operands(A, lda, W_pairs, ldw, M, 2 * I, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!out || !aligned16(out) || ldo % 8 != 0 || ldo < I) return B2_ERR_ARG;
  GemmArgs args{};
  args.C = static_cast<uint16_t*>(out);
  args.ldc = ldo;
  args.silu_pairs = 1;
  return launch_gemm<EPI_STORE>(ctx, A, lda, W_pairs, ldw, M, 2 * I, K, args, 0, static_cast<cudaStream_t>(stream));
}

int b2_rowpar_fused_twoshot(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, int M, int N, int Kr,
                            const void* residual_in, const void* norm_w, float eps, void** normed_out, void* residual_out, void* stream) {
  if (ctx == nullptr || normed_out == nullptr) return B2_ERR_ARG;
  *normed_out = nullptr;
  int rc = check_operands(A, lda, W, ldw, M, N, Kr);
  if (rc != B2_OK) return rc;
  if (ctx->cfg.world < 2) return b2::set_error(B2_ERR_STATE, "b2_rowpar_fused_twoshot needs a tensor-parallel size of 2 or more");
  if (!ctx->peers_ready) return B2_ERR_STATE;
  if (M > ctx->cfg.max_tokens || N != ctx->cfg.hidden || N > MAX_ROW_VECS * NUM_THREADS * 8)
    return b2::set_error(B2_ERR_SHAPE, "b2_rowpar_fused_twoshot: M = %d (limit %d), N = %d (must equal the context's hidden size %d)", M,
                         ctx->cfg.max_tokens, N, ctx->cfg.hidden);
  *normed_out = ctx->symm + ctx->off_out;
  if (M == 0) return B2_OK;
  if (norm_w != nullptr && (!residual_in || !residual_out || !aligned16(residual_in) || !aligned16(residual_out) || !aligned16(norm_w)))
    return B2_ERR_ARG;
  if (bias != nullptr && !aligned16(bias)) return B2_ERR_ARG;
  const int world = ctx->cfg.world;
  GemmArgs args{};
  args.bias = (ctx->cfg.rank == 0) ? static_cast<const uint16_t*>(bias) : nullptr;
  args.rows_per_rank = owned_rows(M, world, 0);
  const size_t max_rows = ((static_cast<size_t>(ctx->cfg.max_tokens) + OWN_ROWS - 1) / OWN_ROWS + world - 1) / world * OWN_ROWS;
  args.slot_stride = max_rows * ctx->cfg.hidden * 2;
  args.parity_stride = args.slot_stride * world;
  for (int r = 0; r < world; ++r) {
    args.inbox[r] = ctx->peer[r] + ctx->off_inbox2;
  }
  args.out_off = ctx->off_out - ctx->off_inbox2;
  args.rowcnt_off = ctx->off_rowcnt - ctx->off_inbox2;
  args.world = world;
  args.rank = ctx->cfg.rank;
  args.residual_in = static_cast<const uint16_t*>(residual_in);
  args.norm_w = static_cast<const uint16_t*>(norm_w);
  args.eps = eps;
  args.residual_out = static_cast<uint16_t*>(residual_out);
  args.dstate = ctx->dstate;
  args.timeout_ns = static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull;
  return launch_gemm<EPI_PUSH2>(ctx, A, lda, W, ldw, M, N, Kr, args, args.rows_per_rank, static_cast<cudaStream_t>(stream));
}

// AUTO: the one-shot form for decode-sized calls (one NVLink store latency; its bytes are few) and at 1 or 2 ranks (one
// copy to send either way).  At 4 ranks and more the row-owner form from owner_min_tokens to owner_max_tokens tokens,
// where sending every partial to every rank and reducing every row on every rank costs more than the second hop and the
// two fences - measured: from 65 tokens at 8 ranks, from 192 at 4 ranks, and only while the rank's K range is short
// enough (<= 6144) for one whole tile per CTA; with a longer K the one-shot form stays ahead up to the two-shot range.
static int auto_form(const b2_ctx* ctx, int m, int kr) {
  const int world = ctx->cfg.world;
  if (world < 4 || m < ctx->owner_min_tokens || m > ctx->owner_max_tokens) return B2_FORM_ONESHOT;
  if ((kr + BK - 1) / BK > 96) return B2_FORM_ONESHOT;
  if (world < 8 && m < 192) return B2_FORM_ONESHOT;
  return B2_FORM_OWNER;
}

// Which form of the fused row-parallel block serves M tokens on this context (B2_FORM_*).
static int rowpar_form_for(const b2_ctx* ctx, int M, int N) {
  const int world = ctx->cfg.world;
  if (world >= 2 && M >= ctx->twoshot_min_tokens && N == ctx->cfg.hidden && M <= ctx->cfg.max_tokens) return B2_FORM_TWOSHOT;
  if (ctx->rowpar_form == B2_FORM_ONESHOT || ctx->rowpar_form == B2_FORM_OWNER) return ctx->rowpar_form;
  return auto_form(ctx, M, 0);  // (without K: the form for a short K range)
}

int b2_rowpar_form(b2_ctx* ctx, int M, int N) {
  if (ctx == nullptr || M < 0 || N <= 0) return -B2_ERR_ARG;
  return rowpar_form_for(ctx, M, N);
}

int b2_ctx_set_option(b2_ctx* ctx, int option, int64_t value) {
  if (ctx == nullptr) return B2_ERR_ARG;
  switch (option) {
    case B2_OPT_ROWPAR_FORM:
      if (value != B2_FORM_AUTO && value != B2_FORM_ONESHOT && value != B2_FORM_OWNER) return B2_ERR_ARG;
      ctx->rowpar_form = static_cast<int>(value);
      return B2_OK;
    case B2_OPT_OWNER_MAX_TOKENS:
      if (value < 0) return B2_ERR_ARG;
      ctx->owner_max_tokens = static_cast<int>(std::min<int64_t>(value, ctx->cfg.oneshot_tokens));
      return B2_OK;
    case B2_OPT_OWNER_MIN_TOKENS:
      if (value < 1) return B2_ERR_ARG;
      ctx->owner_min_tokens = static_cast<int>(std::min<int64_t>(value, 1 << 30));
      return B2_OK;
    case B2_OPT_WHOLE_TILES:
      ctx->whole_tiles = value != 0;
      return B2_OK;
    case B2_OPT_TWOSHOT_MIN_TOKENS:
      if (value < 1) return B2_ERR_ARG;
      ctx->twoshot_min_tokens = static_cast<int>(std::min<int64_t>(value, 1 << 30));
      return B2_OK;
    default:
      return B2_ERR_ARG;
  }
}

int b2_rowpar_fused(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, int M, int N, int Kr,
                    const void* residual_in, const void* norm_w, float eps, void* normed_out, void* residual_out, void* stream) {
  if (ctx == nullptr) return B2_ERR_ARG;
  int rc = check_operands(A, lda, W, ldw, M, N, Kr);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!ctx->peers_ready) return B2_ERR_STATE;
  if (N > ctx->cfg.hidden || N > MAX_ROW_VECS * NUM_THREADS * 8) return B2_ERR_SHAPE;
  if (!normed_out || !aligned16(normed_out)) return B2_ERR_ARG;
  if (norm_w != nullptr && (!residual_in || !residual_out || !aligned16(residual_in) || !aligned16(residual_out) || !aligned16(norm_w)))
    return B2_ERR_ARG;
  if (bias != nullptr && !aligned16(bias)) return B2_ERR_ARG;
  const int chunk = ctx->cfg.oneshot_tokens;
  const int world = ctx->cfg.world;
  if (world == 1 && M > 64 && ctx->rowpar_form == B2_FORM_AUTO) {
    // One rank, many tokens: nothing crosses a link, so the block is the plain GEMM (CTA pairs from 512 tokens on)
    // followed by the HBM-bound add + RMSNorm kernel in place - two launches, both near their rooflines, instead of
    // one whose reduce phase walks the rows one CTA at a time.
    GemmArgs args{};
    args.C = static_cast<uint16_t*>(normed_out);
    args.ldc = N;
    args.bias = static_cast<const uint16_t*>(bias);
    rc = launch_gemm<EPI_STORE>(ctx, A, lda, W, ldw, M, N, Kr, args, 0, static_cast<cudaStream_t>(stream));
    if (rc != B2_OK || norm_w == nullptr) return rc;
    return b2_add_rmsnorm(normed_out, residual_in, norm_w, eps, M, N, normed_out, residual_out, stream);
  }
  for (int m0 = 0; m0 < M; m0 += chunk) {
    const int m = std::min(chunk, M - m0);
    // the owner form when it is cheaper (or forced); every rank decides alike: the choice depends on M and the context only
    int form = ctx->rowpar_form;
    if (form == B2_FORM_AUTO) form = auto_form(ctx, m, Kr);
    GemmArgs args{};
    args.bias = (ctx->cfg.rank == 0) ? static_cast<const uint16_t*>(bias) : nullptr;  // bias enters the sum once
    args.world = world;
    args.rank = ctx->cfg.rank;
    const size_t eoff = static_cast<size_t>(m0) * N;
    args.residual_in = residual_in ? static_cast<const uint16_t*>(residual_in) + eoff : nullptr;
    args.norm_w = static_cast<const uint16_t*>(norm_w);
    args.eps = eps;
    args.normed_out = static_cast<uint16_t*>(normed_out) + eoff;
    args.residual_out = residual_out ? static_cast<uint16_t*>(residual_out) + eoff : nullptr;
    args.dstate = ctx->dstate;
    args.timeout_ns = static_cast<uint64_t>(ctx->cfg.timeout_ms) * 1000000ull;
    const uint16_t* a_rows = static_cast<const uint16_t*>(A) + static_cast<size_t>(m0) * lda;
    if (form == B2_FORM_OWNER) {
      const size_t rows3 = (static_cast<size_t>(ctx->cfg.oneshot_tokens) + world - 1) / world;
      for (int r = 0; r < world; ++r) args.inbox[r] = ctx->peer[r] + ctx->off_inbox3;
      args.slot_stride = rows3 * ctx->cfg.hidden * 2;
      args.parity_stride = args.slot_stride * world;
      args.land_off = ctx->off_land - ctx->off_inbox3;
      args.land_plane_stride = static_cast<size_t>(ctx->cfg.oneshot_tokens) * ctx->cfg.hidden * 2;
      args.land_parity_stride = 2 * args.land_plane_stride;
      rc = launch_gemm<EPI_PUSH3>(ctx, a_rows, lda, W, ldw, m, N, Kr, args, 0, static_cast<cudaStream_t>(stream));
    } else {
      for (int r = 0; r < world; ++r) args.inbox[r] = ctx->peer[r] + ctx->off_rowpar;
      args.slot_stride = static_cast<size_t>(ctx->cfg.oneshot_tokens) * ctx->cfg.hidden * 2;
      args.parity_stride = args.slot_stride * world;
      rc = launch_gemm<EPI_PUSH>(ctx, a_rows, lda, W, ldw, m, N, Kr, args, m, static_cast<cudaStream_t>(stream));
    }
    if (rc != B2_OK) return rc;
  }
  return B2_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// GEMM for callers that must not allocate: the split-tile workspace and the
// arrival counters live in a file-scope device array instead of in a context.
// ---------------------------------------------------------------------------
namespace {

constexpr int STATIC_MAX_TOKENS = 64;    // largest M (token rows): the decode-sized tile, BN <= 64
constexpr int STATIC_MAX_CTAS = 148;     // CTAs that may hold a split tile at once
constexpr int STATIC_MAX_TILES = 4096;   // 128-row output tiles: N <= 524288
constexpr size_t STATIC_COUNTER_BYTES = static_cast<size_t>(STATIC_MAX_TILES) * 4 * sizeof(int);
constexpr size_t STATIC_WS_BYTES = static_cast<size_t>(STATIC_MAX_CTAS) * 2 * 128 * STATIC_MAX_TOKENS * sizeof(float);
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_COUNTER_BYTES + STATIC_WS_BYTES;  // 64 KiB + 9.25 MiB

// Every GPU whose context loads this library carries these bytes until the
// process exits.  Host code must never pass the symbol itself to a kernel: on
// the host the name is only a handle; the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

struct StaticScratch {
  bool ready = false;
  unsigned char* base = nullptr;
  int num_sms = 0;
};
constexpr int STATIC_MAX_DEVICES = 64;
StaticScratch g_static[STATIC_MAX_DEVICES];
std::mutex g_static_mutex;

int static_scratch_for_current_device(StaticScratch** out) {
  int dev = -1;
  B2_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= STATIC_MAX_DEVICES) return b2::set_error(B2_ERR_UNSUPPORTED, "b2_gemm_static_scratch: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticScratch& s = g_static[dev];
  if (!s.ready) {
    void* ptr = nullptr;
    B2_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));  // the address on THIS device
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0)
      return b2::set_error(B2_ERR_CUDA, "b2_gemm_static_scratch: bad device address %p for the static scratch", ptr);
    int sms = 0;
    B2_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    s.base = static_cast<unsigned char*>(ptr);
    s.num_sms = sms;
    s.ready = true;
  }
  *out = &s;
  return B2_OK;
}

}  // namespace

extern "C" int b2_gemm_static_scratch(const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, void* C, int64_t ldc,
                                      int M, int N, int K, void* stream) {
  int rc = check_operands(A, lda, W, ldw, M, N, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!C || !aligned16(C) || ldc % 8 != 0 || ldc < N) return B2_ERR_ARG;
  if (bias != nullptr && !aligned16(bias)) return B2_ERR_ARG;
  if (M > STATIC_MAX_TOKENS)
    return b2::set_error(B2_ERR_SHAPE, "b2_gemm_static_scratch: M = %d exceeds the %d token rows the static scratch is sized for; use b2_gemm",
                         M, STATIC_MAX_TOKENS);
  const int tilesP = (N + BM - 1) / BM;
  if (tilesP > STATIC_MAX_TILES)
    return b2::set_error(B2_ERR_SHAPE, "b2_gemm_static_scratch: N = %d needs %d output tiles, the static scratch holds counters for %d; use b2_gemm",
                         N, tilesP, STATIC_MAX_TILES);
  StaticScratch* sc = nullptr;
  rc = static_scratch_for_current_device(&sc);
  if (rc != B2_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  const int bn = M <= 32 ? 32 : 64;
  GemmArgs args{};
  args.C = static_cast<uint16_t*>(C);
  args.ldc = ldc;
  args.bias = static_cast<const uint16_t*>(bias);
  args.tilesP = tilesP;
  args.tilesQ = 1;
  args.kblocks = (K + BK - 1) / BK;
  args.M = M;
  args.N = N;
  args.counters = reinterpret_cast<int*>(sc->base);
  args.ws = reinterpret_cast<float*>(sc->base + STATIC_COUNTER_BYTES);
  args.status = nullptr;  // no context, hence no status word: an expired pipeline wait only ends the kernel
  args.trace = nullptr;
  const int64_t U = static_cast<int64_t>(tilesP) * args.kblocks;
  if (U > (1ll << 30)) return b2::set_error(B2_ERR_SHAPE, "b2_gemm_static_scratch: problem too large");
  int64_t g = std::max<int64_t>(1, U / 8);
  g = std::min<int64_t>(g, std::min(sc->num_sms, STATIC_MAX_CTAS));
  g = std::min<int64_t>(g, U);
  args.gemm_ctas = static_cast<int>(g);

  // The array keeps whatever the previous call (or an aborted one) left behind.
  // The counters and the accumulation slots of split tiles must start at zero.
  B2_CUDA(cudaMemsetAsync(sc->base, 0, static_cast<size_t>(tilesP) * 4 * sizeof(int), s));
  B2_CUDA(cudaMemsetAsync(sc->base + STATIC_COUNTER_BYTES, 0, static_cast<size_t>(args.gemm_ctas) * 128 * bn * sizeof(float), s));

  CUtensorMap tmP, tmQ;
  rc = b2::encode_tmap_2d(&tmP, W, K, N, ldw, BK, BM);
  if (rc != B2_OK) return rc;
  rc = b2::encode_tmap_2d(&tmQ, A, K, M, lda, BK, bn);
  if (rc != B2_OK) return rc;
  if (bn == 32) return launch_inst<32, true, EPI_STORE>(tmP, tmQ, args, args.gemm_ctas, s);
  return launch_inst<64, true, EPI_STORE>(tmP, tmQ, args, args.gemm_ctas, s);
}

// ---------------------------------------------------------------------------
// The planner as data, for tests that run without a GPU (no CUDA call here).
// ---------------------------------------------------------------------------
static_assert(sizeof(b2_gemm_plan) == sizeof(GemmPlan), "b2_gemm_plan mirrors GemmPlan");

extern "C" int b2_plan_gemm(int epilogue, int M, int N, int K, int num_sms, const int* resident_clusters, b2_gemm_plan* plan) {
  return b2_plan_gemm_opts(epilogue, M, N, K, num_sms, resident_clusters, 0, plan);
}

extern "C" int b2_plan_gemm_opts(int epilogue, int M, int N, int K, int num_sms, const int* resident_clusters, int options,
                                 b2_gemm_plan* plan) {
  if (plan == nullptr || epilogue < EPI_STORE || epilogue > EPI_PUSH3) return B2_ERR_ARG;
  GemmPlan p{};
  const int min_grid = epilogue == EPI_PUSH ? M : 0;  // the one-shot launch also wants a CTA per token row for its reduce phase
  const int rc = plan_gemm(epilogue, M, N, K, num_sms, min_grid, 0, 1 << 20, resident_clusters != nullptr,
                           [&](int bn, int S) { return resident_clusters[(bn == 32 ? 0 : 9) + S]; }, p, options);
  if (rc != B2_OK) return rc;
  plan->swap = p.swap;
  plan->bn = p.bn;
  plan->tiles_p = p.tilesP;
  plan->tiles_q = p.tilesQ;
  plan->kblocks = p.kblocks;
  plan->gemm_ctas = p.gemm_ctas;
  plan->round_robin = p.round_robin;
  plan->grid = p.grid;
  plan->cluster_split = p.cluster_split;
  return B2_OK;
}

extern "C" int b2_plan_cta_units(const b2_gemm_plan* plan, int cta, int* units, int cap) {
  if (plan == nullptr || cta < 0 || cap < 0 || (cap > 0 && units == nullptr)) return -B2_ERR_ARG;
  if (plan->cluster_split > 0) {  // gemm_cluster_kernel: tile = cluster index, K blocks split evenly over the cluster
    const int S = plan->cluster_split, tile = cta / S, crank = cta % S;
    if (tile >= plan->tiles_p * plan->tiles_q) return 0;
    const int base = plan->kblocks / S, rem = plan->kblocks % S;
    const int kb0 = crank * base + (crank < rem ? crank : rem);
    const int n = base + (crank < rem ? 1 : 0);
    for (int i = 0; i < n && i < cap; ++i) {
      units[3 * i] = tile;
      units[3 * i + 1] = kb0 + i;
      units[3 * i + 2] = i == 0 ? 1 : 0;
    }
    return n;
  }
  const int tiles = plan->tiles_p * plan->tiles_q;
  const Work w = make_work(cta, plan->gemm_ctas, tiles, plan->kblocks, plan->round_robin != 0);
  // the producer's walk (Cursor) and the consumers' walk (next_seg) must name the same units in the same order
  Cursor c = cursor_begin(w, plan->tiles_q);
  int i = 0, n = 0;
  Seg s;
  while (next_seg(w, i, s)) {
    for (int kb = s.kb0; kb < s.kb1; ++kb, ++n) {
      if (c.tile != s.tile || c.kb != kb || c.tp != s.tile / plan->tiles_q || c.tq != s.tile % plan->tiles_q) return -B2_ERR_SHAPE;
      if (n < cap) {
        units[3 * n] = s.tile;
        units[3 * n + 1] = kb;
        units[3 * n + 2] = kb == s.kb0 ? 1 : 0;
      }
      cursor_next(w, plan->tiles_q, c);
    }
  }
  return n == w.n_units ? n : -B2_ERR_SHAPE;
}

extern "C" int b2_plan_tile_contributors(const b2_gemm_plan* plan, int tile, int* first_cta, int* last_cta) {
  if (plan == nullptr || first_cta == nullptr || last_cta == nullptr || tile < 0 || tile >= plan->tiles_p * plan->tiles_q) return B2_ERR_ARG;
  if (plan->cluster_split > 0) {
    *first_cta = tile * plan->cluster_split;
    *last_cta = *first_cta + plan->cluster_split - 1;
  } else if (plan->round_robin) {
    *first_cta = *last_cta = tile % plan->gemm_ctas;
  } else {
    const Work w = make_work(0, plan->gemm_ctas, plan->tiles_p * plan->tiles_q, plan->kblocks, false);
    *first_cta = w.part.cta_of(tile * plan->kblocks);
    *last_cta = w.part.cta_of(tile * plan->kblocks + plan->kblocks - 1);
  }
  return B2_OK;
}

extern "C" int b2_last_gemm_kernel(void) { return g_last_gemm_path; }

extern "C" int b2_row_owner(int token, int world, int* local_row) {
  if (token < 0 || world < 1 || local_row == nullptr) return -B2_ERR_ARG;
  return owner_of(token, world, *local_row);
}

extern "C" int b2_owner_form_row(int token, int world, int* local_row) {
  if (token < 0 || world < 1 || local_row == nullptr) return -B2_ERR_ARG;
  return owner3_of(token, world, *local_row);
}

extern "C" int b2_owner_form_rows(int M, int world, int rank) {
  if (M < 0 || world < 1 || rank < 0 || rank >= world) return -B2_ERR_ARG;
  return owned_rows3(M, world, rank);
}

extern "C" int b2_owned_rows(int M, int world, int rank) {
  if (M < 0 || world < 1 || rank < 0 || rank >= world) return -B2_ERR_ARG;
  return owned_rows(M, world, rank);
}
