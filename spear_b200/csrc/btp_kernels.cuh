// BTP forward and backward kernels for sm_100a.
//
// What is computed (per (b,h) sequence, 16 channels, blocks of 16 tokens; semantics of
// spear/ops/btp/reference.py:105-139 and csrc/btp/btp-forward.cu:85-457,
// csrc/btp/btp-backwards.cu:165-808):
//   T_r       = sum_{j<=r} log2 a_j                      (inclusive, per block)
//   Lmat[r,c] = 2^(T_r - T_c) for c <= r, else 0         P[r] = 2^(T_r)
//   v_i       = x_i . Lmat^T                             (local pass, tensor cores)
//   y_i       = v_i + P (x) carry_i,   carry_i = v_{i-1}[:,15]   (ONE hop, never the corrected value)
//   gw_i      = dy_i . Lmat,  dCarry_i = P[0] gw_i[:,0]
//   dx_i[:,c] = gw_i[:,c] + Lmat[15,c] dCarry_{i+1}
//   dA_i[t]   = sum_ch v_i[ch,t-1] dx_i[ch,t] + P[t-1] sum_ch gw_i[ch,t] carry_i[ch]
//               (v[:, -1] = 0, P[-1] = 1; no division by a anywhere)
//
// How it is mapped to the machine:
//   * Work unit = a chunk of TL = 64*NBOX tokens of one sequence: x as NBOX TMA boxes of
//     [16 channels x 64 tokens] bf16 (128-byte swizzle), the coefficients as one bulk copy.
//   * Every WARP owns a private ring of STAGES chunk buffers with its own mbarriers and walks its
//     own list of chunks (backward: whole sequences dealt round-robin when there are many, else a
//     contiguous range; forward: short runs of chunks dealt round-robin, so that the whole GPU works on
//     one small moving window of memory).  No block-wide or grid-wide synchronisation exists, so no
//     warp ever waits for another warp; the only waits are on the warp's own TMA loads (bounded) and
//     on the previous kernel of the stream (griddepcontrol.wait, see the launch code).  The one exception
//     is the forward's optional HANDOFF variant (SeamLink below), where a warp waits, bounded as well, for
//     the carry its left neighbour hands over inside a thread-block cluster.
//   * Once per chunk the warp turns the coefficients into the per-token tables the blocks need
//     (T, P, and for backward P shifted by one token and the last Lmat row), so that the per-block
//     work is the Lmat fragment (6 exponentials per lane), the tensor-core products and FMAs.
//   * Lmat goes to the tensor cores as two bf16 terms (hi + lo), which reproduces the fp32 matrix to
//     ~2^-17; the per-block fp32 arithmetic of the backward uses packed fp32x2 instructions.
//   * The carry stays in registers while a warp walks along a sequence.  Where a warp's range
//     starts (ends) inside a sequence the neighbouring block is re-read from global memory
//     (16x16 values, a "halo") and its carry (dCarry) recomputed, so no seam ever drops a carry.
//   * The plain backward deals whole sequences from the end of the batch; its TMA stores and the forward's
//     mark their lines to leave L2 last (the outputs are what the next kernel reads).
//   * Outputs in bf16 are written over the consumed input tile in shared memory and leave with a
//     TMA store; fp32 outputs are stored straight from the accumulator fragments (32-byte runs).
#pragma once

#include "btp_ptx.cuh"

namespace btp {

constexpr int kCoefBf16 = 0;    // linear coefficient in the activations' 16-bit type (bf16, or fp16 for the fp16 kernels)
constexpr int kCoefF32 = 1;     // linear coefficient, float
constexpr int kCoefF32Log = 2;  // natural-log coefficient, float

constexpr float kLog2E = 1.4426950408889634f;
constexpr float kZeroLog2 = -200.0f;  // stands in for log2(0): 2^-200 flushes to zero, sums stay finite
constexpr float kTinyCoeff = 1e-9f;   // coefficients at or below this count as zero (btp-forward.cu:179)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // default: bounded waits give up after 2 s

// Error word written when a bounded wait gives up: {code, blockIdx.x, warp, chunk}.
__device__ unsigned int g_btp_device_error[4];

struct KernelParams {
  const void* coeff;   // [BH, L]
  const void* x;       // [BH*16, L] bf16   (halo reads)
  const void* dy;      // backward: [BH*16, L] (halo reads)
  void* out_f32;       // forward with fp32 output: y
  float* ckpt;         // forward: optional carry checkpoint [BH, L/16, 16]
  float* dA;           // backward: [BH, L]
  int L;               // tokens per sequence
  int ncs;             // chunks per sequence
  int total_chunks;    // BH * ncs
  int use_carry;       // k == 2
  int interleave;      // deal whole sequences round-robin to the warps (short sequences)
  int run_len;         // forward only: > 0 deals runs of this many chunks round-robin (divides ncs); see RunCursor
  unsigned long long wait_limit_ns;  // bounded waits give up after this long (btp_sm100_set_wait_limit)
  unsigned int test_missing_tx;      // test hook: warp 0 of block 0 expects this many bytes that never arrive
};

template <int COEF>
struct CoefTraits {
  static constexpr int kBytes = (COEF == kCoefBf16) ? 2 : 4;
};

// log2 of one coefficient as the kernels use it.
template <int COEF>
__device__ __forceinline__ float coef_log2(float a) {
  if constexpr (COEF == kCoefF32Log) {
    return fmaxf(a * kLog2E, kZeroLog2);
  } else {
    return (a > kTinyCoeff) ? lg2(a) : kZeroLog2;
  }
}

// Shared-memory carve-up of one CTA.  Every warp owns
//   * STAGES buffers for the x tiles of a chunk (NBOX boxes of [16][64] bf16, 128-byte swizzled); a bf16
//     output (y, dx) is written over them and leaves from there,
//   * backward: STAGES-1 buffers for the dy tiles (they are dead as soon as the chunk's products are done),
//   * landing zones for the raw coefficients (backward: STAGES; forward: one more than the loads run ahead, the
//     coefficients being consumed at the start of a chunk), backward: STAGES staging rows for dA,
//   * the per-token float tables of the chunk in work (forward: T, P; backward, double-buffered because a
//     chunk's last block is finished one block into the next chunk: T, Pshift, L15).  Forward with float
//     coefficients: the T table is written over the chunk's raw coefficients (same size), which is what lets four
//     CTAs of that kernel share an SM,
//   * STAGES mbarriers.
template <int COEF, int NBOX, int STAGES, int WARPS, bool BWD, bool DY_F32, bool OUT_F32 = false>
struct SmemLayout {
  static constexpr int kTL = 64 * NBOX;                 // tokens per chunk
  static constexpr int kTiles = kTL / 16;               // 16-token blocks per chunk
  static constexpr int kXBytes = NBOX * 2048;
  static constexpr int kDyBytes = BWD ? (DY_F32 ? NBOX * 4096 : NBOX * 2048) : 0;
  static constexpr int kDyStages = BWD ? STAGES - 1 : 0;
  static constexpr int kBigPerWarp = STAGES * kXBytes + kDyStages * kDyBytes;  // multiple of 1024 (swizzle atom)
  static constexpr int kRawBytes = kTL * CoefTraits<COEF>::kBytes;
  static constexpr int kDaBytes = BWD ? kTL * 4 : 0;
  static constexpr int kRawStages = BWD ? STAGES : (OUT_F32 ? STAGES : STAGES - 1);
  static constexpr bool kTInPlace = !BWD && COEF != kCoefBf16;
  static constexpr int kTabFloats = (BWD ? 3 : (kTInPlace ? 1 : 2)) * kTL;
  static constexpr int kTabSets = BWD ? 2 : 1;
  static constexpr int kSmallPerWarp = kRawStages * kRawBytes + STAGES * kDaBytes + kTabSets * kTabFloats * 4;
  static constexpr int kBarsPerWarp = STAGES * 8;
  static constexpr int kBytes = WARPS * (kBigPerWarp + kSmallPerWarp + kBarsPerWarp);
};

// Per-warp view of its buffers (shared-space addresses for the async copies, generic pointers for the tables).
template <class LAYOUT, int STAGES>
struct WarpSmem {
  uint32_t big, small, bars;
  unsigned char* small_ptr;
  __device__ __forceinline__ uint32_t x(int s) const { return big + s * LAYOUT::kXBytes; }
  __device__ __forceinline__ uint32_t dy(int d) const { return big + STAGES * LAYOUT::kXBytes + d * LAYOUT::kDyBytes; }
  __device__ __forceinline__ uint32_t raw_addr(int s) const { return small + s * LAYOUT::kRawBytes; }
  __device__ __forceinline__ void* raw_ptr(int s) const { return small_ptr + s * LAYOUT::kRawBytes; }
  __device__ __forceinline__ uint32_t da_addr(int s) const {
    return small + LAYOUT::kRawStages * LAYOUT::kRawBytes + s * LAYOUT::kDaBytes;
  }
  __device__ __forceinline__ float* da_ptr(int s) const {
    return reinterpret_cast<float*>(small_ptr + LAYOUT::kRawStages * LAYOUT::kRawBytes + s * LAYOUT::kDaBytes);
  }
  __device__ __forceinline__ float* tab_ptr(int set) const {
    return reinterpret_cast<float*>(small_ptr + LAYOUT::kRawStages * LAYOUT::kRawBytes + STAGES * LAYOUT::kDaBytes +
                                    set * LAYOUT::kTabFloats * 4);
  }
  __device__ __forceinline__ uint32_t bar(int s) const { return bars + s * 8; }
};

template <class LAYOUT, int STAGES, int WARPS>
__device__ __forceinline__ WarpSmem<LAYOUT, STAGES> carve_smem(unsigned char* raw, int warp) {
  const uint32_t base = smem_u32(raw);
  WarpSmem<LAYOUT, STAGES> w;
  w.big = base + warp * LAYOUT::kBigPerWarp;
  w.small = base + WARPS * LAYOUT::kBigPerWarp + warp * LAYOUT::kSmallPerWarp;
  w.small_ptr = raw + WARPS * LAYOUT::kBigPerWarp + warp * LAYOUT::kSmallPerWarp;
  w.bars = base + WARPS * (LAYOUT::kBigPerWarp + LAYOUT::kSmallPerWarp) + warp * LAYOUT::kBarsPerWarp;
  return w;
}

// One lane's share of a chunk's asynchronous copies.  The copies of a chunk (its x boxes, its dy boxes, its row of
// coefficients; on the way out its dx boxes and its row of dA) are all 2-D tiled copies that differ only in
// descriptor, shared-memory address and coordinates.  Lane i of the warp keeps copy i's parameters in its own
// registers and all the lanes concerned execute ONE copy instruction together, instead of one lane issuing
// them one after the other: the per-chunk producer code shrinks to a handful of warp instructions.
struct LaneCopy {
  uint64_t map;    // generic address of the descriptor (a __grid_constant__ kernel parameter)
  uint32_t cur;    // shared-memory address in the ring's current stage
  uint32_t first;  // ... in stage 0
  uint32_t end;    // first + stages * stride
  uint32_t stride; // bytes from one stage to the next
  int col_off;     // added to the chunk's first token
  int row_mul;     // row coordinate = sequence index * row_mul (16 channel rows, or 1 row of coefficients)
  __device__ __forceinline__ void set(const void* m, uint32_t first_, uint32_t stride_, int stages, int col, int rows) {
    map = reinterpret_cast<uint64_t>(m);
    cur = first = first_;
    stride = stride_;
    end = first_ + stages * stride_;
    col_off = col;
    row_mul = rows;
  }
  __device__ __forceinline__ void advance() {
    cur += stride;
    if (cur == end) cur = first;
  }
  __device__ __forceinline__ uint32_t at(int stage) const { return first + stage * stride; }
};

// Position of a chunk; walks forward one chunk at a time (no division after the first).
struct ChunkCursor {
  int bh;    // sequence index
  int cs;    // chunk index inside the sequence
  int step;  // distance, in sequences, from one sequence of this warp to its next
  __device__ __forceinline__ ChunkCursor(int bh_, int cs_, int step_) : bh(bh_), cs(cs_), step(step_) {}
  __device__ __forceinline__ void next(int ncs) {
    if (++cs == ncs) {
      cs = 0;
      bh += step;
    }
  }
};

// Which chunks a warp works on (backward and the gated kernels; the forward kernel uses RunCursor below).
//   Long sequences (or too few of them to balance): a contiguous range of the (sequence, chunk) list, so
//   that the carry runs along the sequence in registers and only the two ends of the range need a halo.
//   Short sequences: whole sequences dealt round-robin to the warps, so that at any moment the whole GPU
//   reads and writes one moving window of memory (measurably kinder to HBM than 2368 separate streams).
//   `from_end`: the window starts at the LAST sequence and moves down.  The plain backward does that: when its
//   forward ran just before it (the training step of the op alone, or a forward recomputed for the backward), the
//   end of x is what L2 still holds (step 1 % faster; nothing changes otherwise).
struct WarpWork {
  int bh, cs;  // first chunk
  int n;       // number of chunks
  int step;    // sequences between consecutive sequences of this warp
  __device__ __forceinline__ WarpWork(long long wid, long long nwarps, int total, int ncs, bool interleave,
                                      bool from_end = false) {
    if (interleave) {
      const long long nseq = total / ncs;
      bh = static_cast<int>(from_end ? nseq - 1 - wid : wid);
      cs = 0;
      step = from_end ? -static_cast<int>(nwarps) : static_cast<int>(nwarps);
      n = wid < nseq ? static_cast<int>((nseq - wid + nwarps - 1) / nwarps) * ncs : 0;
    } else {
      const int first = static_cast<int>((wid * total) / nwarps);
      n = static_cast<int>(((wid + 1) * total) / nwarps) - first;
      bh = first / ncs;
      cs = first - bh * ncs;
      step = 1;
    }
  }
};

// Forward work list with a third mode between the two of WarpWork: RUNS of `run_len` consecutive chunks of a
// sequence are dealt round-robin to the warps.  Few long sequences then still give every warp many units, the
// whole GPU still reads one moving window of memory, and a carry has to be recomputed only once per run.
//   run_len == ncs  : whole sequences round-robin (no halo at all)
//   run_len  < ncs  : runs round-robin, a left halo at the start of every run that is not a sequence start
//   run_len == 0    : one contiguous range per warp (halo at its first chunk only)
struct RunCursor {
  int bh, cs;        // current chunk
  int left;          // chunks left in the current run, this one included (contiguous mode: never reaches 0)
  int q;             // index of the current run inside its sequence
  int rps, len;      // runs per sequence, chunks per run
  int dbh, dq;       // the warp's next run lies dbh sequences and dq runs further on (no division per run)
  bool fresh;        // the current chunk starts a run (or the warp's range)
  __device__ __forceinline__ void next(int ncs) {
    fresh = false;
    if (--left == 0) {
      bh += dbh;
      q += dq;
      if (q >= rps) {
        q -= rps;
        ++bh;
      }
      cs = q * len;
      left = len;
      fresh = true;
    } else if (++cs == ncs) {  // only a contiguous range crosses from one sequence into the next
      cs = 0;
      ++bh;
    }
  }
};

// n = number of chunks of warp `wid`; `c` is left on its first chunk.
__device__ __forceinline__ int forward_work(long long wid, long long nwarps, const KernelParams& p, RunCursor& c) {
  c.fresh = true;
  if (p.run_len > 0) {
    c.len = p.run_len;
    c.rps = p.ncs / p.run_len;
    const long long total_runs = static_cast<long long>(p.total_chunks) / p.run_len;
    if (wid >= total_runs) return 0;
    c.bh = static_cast<int>(wid / c.rps);
    c.q = static_cast<int>(wid - static_cast<long long>(c.bh) * c.rps);
    c.dbh = static_cast<int>(nwarps / c.rps);
    c.dq = static_cast<int>(nwarps - static_cast<long long>(c.dbh) * c.rps);
    c.cs = c.q * c.len;
    c.left = c.len;
    return static_cast<int>((total_runs - wid + nwarps - 1) / nwarps) * p.run_len;
  }
  const int first = static_cast<int>((wid * p.total_chunks) / nwarps);
  const int n = static_cast<int>(((wid + 1) * p.total_chunks) / nwarps) - first;
  c.bh = first / p.ncs;
  c.cs = first - c.bh * p.ncs;
  c.left = 0x7fffffff;
  c.q = c.dbh = c.dq = 0;
  c.rps = c.len = 1;
  return n;
}

// Blocks in chunk `cs`.  RAGGED == false: L is a multiple of the chunk width, every chunk is full and
// the count folds to a constant.
template <int TL, bool RAGGED>
__device__ __forceinline__ int chunk_tiles(int cs, int L) {
  if constexpr (!RAGGED) {
    return TL / 16;
  } else {
    const int left = (L - cs * TL) >> 4;
    return left < TL / 16 ? left : TL / 16;
  }
}

// Tables of one chunk from the log2 of its coefficients, held in registers: lane l owns TPL = TL/32
// consecutive tokens, 16/TPL lanes make one block, the prefix sums restart at every block.
// Tables (each TL floats): [0] T, then forward [1] P = 2^T,
// backward [1] Pshift (P of the previous token, 1 for the first token of a block), [2] L15 = 2^(T_15 - T).
// `carry_scale` is 1 (k = 2) or 0 (k = 1): every use of the carry and of the gradient that flows back
// through it is multiplied by an entry of the P / Pshift table, so zeroing that table switches the one-hop
// term off without a single extra instruction per block.
// Destinations: tab = T; tab2 = the second table; the third (backward only) follows the second.
template <int TL, bool BWD>
__device__ __forceinline__ void tables_from_log2(const float (&l2)[TL / 32], float* tab, float* tab2, int lane,
                                                 float carry_scale) {
  constexpr int TPL = TL / 32;    // tokens per lane: 1, 2 or 4
  constexpr int LPT = 16 / TPL;   // lanes per block: 16, 8 or 4
  float T[TPL];
  T[0] = l2[0];
#pragma unroll
  for (int k = 1; k < TPL; ++k) T[k] = T[k - 1] + l2[k];
  // exclusive prefix of the lane totals inside the block
  const int q = lane & (LPT - 1);
  float inc = T[TPL - 1];
#pragma unroll
  for (int d = 1; d < LPT; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, inc, d, LPT);
    if (q >= d) inc += up;
  }
  float excl = __shfl_up_sync(0xffffffffu, inc, 1, LPT);
  if (q == 0) excl = 0.0f;
  float P[TPL];
#pragma unroll
  for (int k = 0; k < TPL; ++k) {
    T[k] += excl;
    P[k] = ex2(T[k]);
  }
  float second[TPL], third[TPL];
  if constexpr (BWD) {
    const float T15 = __shfl_sync(0xffffffffu, T[TPL - 1], lane | (LPT - 1));
    float prev = __shfl_up_sync(0xffffffffu, P[TPL - 1], 1, LPT);
    if (q == 0) prev = 1.0f;
    second[0] = prev * carry_scale;
#pragma unroll
    for (int k = 1; k < TPL; ++k) second[k] = P[k - 1] * carry_scale;
#pragma unroll
    for (int k = 0; k < TPL; ++k) third[k] = ex2(T15 - T[k]);
  } else {
#pragma unroll
    for (int k = 0; k < TPL; ++k) {
      second[k] = P[k] * carry_scale;
      third[k] = 0.0f;
    }
  }
  __syncwarp();  // nobody still reads the tables of the chunk before
  if constexpr (TPL == 4) {
    reinterpret_cast<float4*>(tab)[lane] = make_float4(T[0], T[1], T[2], T[3]);
    reinterpret_cast<float4*>(tab2)[lane] = make_float4(second[0], second[1], second[2], second[3]);
    if constexpr (BWD) reinterpret_cast<float4*>(tab2 + TL)[lane] = make_float4(third[0], third[1], third[2], third[3]);
  } else if constexpr (TPL == 2) {
    reinterpret_cast<float2*>(tab)[lane] = make_float2(T[0], T[1]);
    reinterpret_cast<float2*>(tab2)[lane] = make_float2(second[0], second[1]);
    if constexpr (BWD) reinterpret_cast<float2*>(tab2 + TL)[lane] = make_float2(third[0], third[1]);
  } else {
    tab[lane] = T[0];
    tab2[lane] = second[0];
    if constexpr (BWD) tab2[TL + lane] = third[0];
  }
  __syncwarp();
}

// Once per chunk: raw coefficients (already in shared memory at `rawp`) -> per-token tables: T at `tab`, the others
// from `tab2` on.  `tab` may be `rawp` itself when the coefficients are floats: a lane reads exactly the elements it
// writes, and reads them first.
template <int COEF, int TL, bool BWD, bool F16 = false>
__device__ __forceinline__ void chunk_tables(const void* rawp, float* tab, float* tab2, int lane, float carry_scale) {
  constexpr int TPL = TL / 32;  // tokens per lane: 2 or 4
  float v[TPL];
  if constexpr (COEF == kCoefBf16) {
    if constexpr (TPL == 4) {
      const uint2 raw = reinterpret_cast<const uint2*>(rawp)[lane];
      v[0] = Act<F16>::lo(raw.x); v[1] = Act<F16>::hi(raw.x); v[2] = Act<F16>::lo(raw.y); v[3] = Act<F16>::hi(raw.y);
    } else {
      const uint32_t raw = reinterpret_cast<const uint32_t*>(rawp)[lane];
      v[0] = Act<F16>::lo(raw); v[1] = Act<F16>::hi(raw);
    }
  } else {
    if constexpr (TPL == 4) {
      const float4 raw = reinterpret_cast<const float4*>(rawp)[lane];
      v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    } else {
      const float2 raw = reinterpret_cast<const float2*>(rawp)[lane];
      v[0] = raw.x; v[1] = raw.y;
    }
  }
  float l2[TPL];
#pragma unroll
  for (int k = 0; k < TPL; ++k) l2[k] = coef_log2<COEF>(v[k]);
  tables_from_log2<TL, BWD>(l2, tab, tab2, lane, carry_scale);
}

// Halo: a 16x16 block that belongs to a neighbouring warp's range is read straight from global
// memory and reduced to the 16 numbers the seam needs.
//   LEFT  (RIGHT == false): carry  = sum_c  x[ch,c] * w(2^(T_15 - T_c))             (= v[:,15])
//   RIGHT (RIGHT == true) : dCarry = 2^(T_0) * sum_r dy[ch,r] * w(2^(T_r - T_0))
// w() represents a weight exactly like the Lmat operand of the tensor-core path: one bf16 term, or two
// (hi + lo) when PRECISE.
// Returns the values for channels g and g+8 (g = lane >> 2), identical in the 4 lanes of a group.
template <int COEF, bool TILE_F32, bool RIGHT, bool PRECISE, bool F16 = false>
__device__ __forceinline__ void halo_reduce(const void* tile_base, const void* coeff_base, int L, long long bh,
                                            int tok0, int lane, float& out_g, float& out_g8) {
  const int g = lane >> 2, t = lane & 3;
  float a;
  if constexpr (COEF == kCoefBf16) {
    a = Act<F16>::scalar(reinterpret_cast<const unsigned short*>(coeff_base)[bh * L + tok0 + (lane & 15)]);
  } else {
    a = reinterpret_cast<const float*>(coeff_base)[bh * L + tok0 + (lane & 15)];
  }
  float T = coef_log2<COEF>(a);
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, T, d, 16);
    if ((lane & 15) >= d) T += up;
  }
  const float Tref = __shfl_sync(0xffffffffu, T, RIGHT ? 0 : 15);
  float w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tok = 2 * t + (j & 1) + ((j >> 1) << 3);
    const float Tj = __shfl_sync(0xffffffffu, T, tok);
    w[j] = act_weight<F16, PRECISE>(ex2(RIGHT ? (Tj - Tref) : (Tref - Tj)));
  }
  float e[2][4];  // [row half][token]
  const long long row_g = (bh * 16 + g) * static_cast<long long>(L) + tok0;
  const long long row_g8 = row_g + 8ll * L;
  if constexpr (TILE_F32) {
    const float* p = reinterpret_cast<const float*>(tile_base);
    const float2 a0 = *reinterpret_cast<const float2*>(p + row_g + 2 * t);
    const float2 a1 = *reinterpret_cast<const float2*>(p + row_g + 8 + 2 * t);
    const float2 b0 = *reinterpret_cast<const float2*>(p + row_g8 + 2 * t);
    const float2 b1 = *reinterpret_cast<const float2*>(p + row_g8 + 8 + 2 * t);
    // what the tensor-core path feeds: dy as one bf16 term, or as two (hi + lo) when PRECISE
    e[0][0] = act_weight<F16, PRECISE>(a0.x); e[0][1] = act_weight<F16, PRECISE>(a0.y);
    e[0][2] = act_weight<F16, PRECISE>(a1.x); e[0][3] = act_weight<F16, PRECISE>(a1.y);
    e[1][0] = act_weight<F16, PRECISE>(b0.x); e[1][1] = act_weight<F16, PRECISE>(b0.y);
    e[1][2] = act_weight<F16, PRECISE>(b1.x); e[1][3] = act_weight<F16, PRECISE>(b1.y);
  } else {
    const unsigned short* p = reinterpret_cast<const unsigned short*>(tile_base);
    const uint32_t a0 = *reinterpret_cast<const uint32_t*>(p + row_g + 2 * t);
    const uint32_t a1 = *reinterpret_cast<const uint32_t*>(p + row_g + 8 + 2 * t);
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(p + row_g8 + 2 * t);
    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(p + row_g8 + 8 + 2 * t);
    e[0][0] = Act<F16>::lo(a0); e[0][1] = Act<F16>::hi(a0); e[0][2] = Act<F16>::lo(a1); e[0][3] = Act<F16>::hi(a1);
    e[1][0] = Act<F16>::lo(b0); e[1][1] = Act<F16>::hi(b0); e[1][2] = Act<F16>::lo(b1); e[1][3] = Act<F16>::hi(b1);
  }
  float sg = 0.0f, sg8 = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    sg = fmaf(e[0][j], w[j], sg);
    sg8 = fmaf(e[1][j], w[j], sg8);
  }
  sg += __shfl_xor_sync(0xffffffffu, sg, 1);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 1);
  sg += __shfl_xor_sync(0xffffffffu, sg, 2);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 2);
  if constexpr (RIGHT) {
    const float a0 = ex2(Tref);
    sg *= a0;
    sg8 *= a0;
  }
  out_g = sg;
  out_g8 = sg8;
}

// Lane-constant pieces of the addressing of 16x16 bf16 blocks inside 128-byte-swizzled [16][64] boxes.
// Block ib (0..3) of a box occupies the 16-byte columns 2*ib and 2*ib+1 of every 128-byte row; the
// hardware swizzle stores column c of row r at column c ^ (r & 7).
struct TileLane {
  int g, t;
  uint32_t ldm_base;    // ldmatrix: byte offset of this lane's row
  uint32_t ldm_off[4];  // ldmatrix: swizzled column offset for ib = 0..3
  uint32_t st_base;     // fragment store: byte offset of (channel g, tokens 2t..2t+1)
  uint32_t st_off[4];   // fragment store: swizzled column offset of the first token half, ib = 0..3
  bool m0, m1;          // 2t <= g, 2t+1 <= g  (causal mask of the fragment elements)
  __device__ __forceinline__ explicit TileLane(int lane) {
    g = lane >> 2;
    t = lane & 3;
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t key = (lane >> 4) ^ (row & 7);
    ldm_base = row * 128;
    st_base = g * 128 + t * 4;
#pragma unroll
    for (int ib = 0; ib < 4; ++ib) {
      ldm_off[ib] = ((2u * ib) ^ key) << 4;
      st_off[ib] = ((2u * ib) ^ static_cast<uint32_t>(g)) << 4;
    }
    m0 = (2 * t) <= g;
    m1 = (2 * t + 1) <= g;
  }
};

// Lmat fragments of one block for the local pass v = x . Lmat^T  (B operand: k = c, n = r).
struct LmatFrag {
  uint32_t b00;  // rows 0..7  x cols 0..7
  uint32_t b10;  // rows 8..15 x cols 0..7
  uint32_t b11;  // rows 8..15 x cols 8..15
};

// tg = &T[g], tt = &T[2t] of the chunk; `off` = 16 * block index (a compile-time constant in the hot loops)
template <bool F16 = false>
__device__ __forceinline__ LmatFrag build_lmat(const float* tg, const float* tt, int off, const TileLane& tl) {
  const float Tg = tg[off];
  const float Tg8 = tg[off + 8];
  const float2 Ta = *reinterpret_cast<const float2*>(tt + off);
  const float2 Tb = *reinterpret_cast<const float2*>(tt + off + 8);
  const float e0 = tl.m0 ? ex2(Tg - Ta.x) : 0.0f;
  const float e1 = tl.m1 ? ex2(Tg - Ta.y) : 0.0f;
  const float e2 = ex2(Tg8 - Ta.x);
  const float e3 = ex2(Tg8 - Ta.y);
  const float e4 = tl.m0 ? ex2(Tg8 - Tb.x) : 0.0f;
  const float e5 = tl.m1 ? ex2(Tg8 - Tb.y) : 0.0f;
  LmatFrag f;
  f.b00 = Act<F16>::pack(e0, e1);
  f.b10 = Act<F16>::pack(e2, e3);
  f.b11 = Act<F16>::pack(e4, e5);
  return f;
}

// code 1: a bounded wait gave up; code 2: shared-memory base not 1024-byte aligned
// The same fragments split into two bf16 terms, Lmat = hi + lo with |lo| <= 2^-9 |hi|: feeding both to the
// tensor cores reproduces the fp32 Lmat to about 2^-17 instead of 2^-9.
template <bool F16 = false>
__device__ __forceinline__ void build_lmat_split(const float* tg, const float* tt, int off, const TileLane& tl,
                                                 LmatFrag& hi, LmatFrag& lo) {
  using A = Act<F16>;
  const float Tg = tg[off];
  const float Tg8 = tg[off + 8];
  const float2 Ta = *reinterpret_cast<const float2*>(tt + off);
  const float2 Tb = *reinterpret_cast<const float2*>(tt + off + 8);
  const float e0 = tl.m0 ? ex2(Tg - Ta.x) : 0.0f;
  const float e1 = tl.m1 ? ex2(Tg - Ta.y) : 0.0f;
  const float e2 = ex2(Tg8 - Ta.x);
  const float e3 = ex2(Tg8 - Ta.y);
  const float e4 = tl.m0 ? ex2(Tg8 - Tb.x) : 0.0f;
  const float e5 = tl.m1 ? ex2(Tg8 - Tb.y) : 0.0f;
  hi.b00 = A::pack(e0, e1);
  hi.b10 = A::pack(e2, e3);
  hi.b11 = A::pack(e4, e5);
  lo.b00 = A::pack(e0 - A::lo(hi.b00), e1 - A::hi(hi.b00));
  lo.b10 = A::pack(e2 - A::lo(hi.b10), e3 - A::hi(hi.b10));
  lo.b11 = A::pack(e4 - A::lo(hi.b11), e5 - A::hi(hi.b11));
}

__device__ __forceinline__ void report_error(unsigned int code, int warp, int chunk) {
  if (atomicCAS(&g_btp_device_error[0], 0u, code) == 0u) {
    g_btp_device_error[1] = blockIdx.x;
    g_btp_device_error[2] = warp;
    g_btp_device_error[3] = chunk;
  }
}

// Hand-off of the carry between the runs of one sequence (forward kernel, HANDOFF).
//
// Runs are dealt round-robin to the warps of the grid and the grid holds a whole number of sequences' worth of
// warps, so a warp always works on run q = (its index) mod (runs per sequence) of some sequence, and the warps with
// the neighbouring indices work on the neighbouring runs of the SAME sequence at the same time.  The launch puts the
// warps of one sequence into one thread-block cluster, so a warp can write into its right neighbour's shared memory.
//   * The carry into a run's first block is only needed for that block's OUTPUT (the carry is one hop: the next
//     block takes the uncorrected last token).  The warp therefore runs through its run without it, keeps the first
//     block's uncorrected result in registers, and corrects and stores that one block at the end of the run.
//   * At the end of its run a warp has the uncorrected last token of the run in registers: exactly what the right
//     neighbour is missing.  It stores the 16 numbers into the neighbour's landing slot (st.async counts the bytes
//     on the neighbour's mbarrier), then waits (bounded) for its own slot to fill.
//   * Two slots per warp, used alternately; before a slot is written a second time the writer waits (bounded) for the
//     credit the reader sends when it has read the slot (an arrive on an mbarrier of the writer).
//   * A warp that gives up (a bounded wait ran out) sets an abort word in every CTA of its cluster; the waits for
//     a hand-off or a credit look at their CTA's word and give up with it, so that one failure ends the kernel
//     after one wait limit, not after one limit per warp of the chain.
// Per warp: 2 x 64 bytes of landing slots, 2 "slot full" barriers, 2 "credit" barriers; per CTA: the abort word.
constexpr int kSeamBytesPerWarp = 2 * 64 + 2 * 8 + 2 * 8;
constexpr int kSeamBytesPerCta = 16;
struct SeamLink {
  uint32_t slot;        // own landing slots (shared::cta address), 64 bytes each: [g][2] floats = channels g, g+8
  uint32_t full;        // own "slot full" barriers
  uint32_t credit;      // own credit barriers (the right neighbour arrives on them)
  uint32_t right_slot;  // right neighbour's landing slots / "slot full" barriers, left neighbour's credit barriers
  uint32_t right_full;  //   (cluster-wide shared addresses)
  uint32_t left_credit;
  uint32_t abort_word;  // own CTA's abort word (shared::cta address)
  __device__ __forceinline__ void set(uint32_t seam_base, int warp, int warps) {
    abort_word = seam_base + static_cast<uint32_t>(warps) * kSeamBytesPerWarp;
    const uint32_t rank = cluster_cta_rank();
    const auto at = [&](int w) { return seam_base + static_cast<uint32_t>(w) * kSeamBytesPerWarp; };
    slot = at(warp);
    full = slot + 128;
    credit = slot + 144;
    const int rw = warp + 1 == warps ? 0 : warp + 1, lw = warp == 0 ? warps - 1 : warp - 1;
    // a warp without a neighbour on that side never uses the address; its rank is clamped so that it stays mappable
    const uint32_t last = cluster_cta_count() - 1;
    const uint32_t rr = warp + 1 == warps ? (rank < last ? rank + 1 : rank) : rank;
    const uint32_t lr = warp == 0 ? (rank > 0 ? rank - 1 : rank) : rank;
    right_slot = map_to_cta(at(rw), rr);
    right_full = right_slot + 128;
    left_credit = map_to_cta(at(lw) + 144, lr);
  }
};

// =====================================================================================
// Forward
// =====================================================================================
// PRECISE: Lmat goes to the tensor cores as two bf16 terms (see build_lmat_split).
// F16: activations (x, y, a 16-bit coefficient) are float16 instead of bfloat16.
// HANDOFF: the carry that crosses the seam between two runs of a sequence is handed from the warp that owns the
// left run to the warp that owns the right one through (distributed) shared memory instead of being recomputed
// from a halo block; see SeamLink.  The kernel is then launched in clusters of runs_per_sequence / WARPS CTAs.
template <int COEF, bool OUT_F32, bool CKPT, bool RAGGED, bool PRECISE, int NBOX, int STAGES, int WARPS, bool F16 = false,
          bool HANDOFF = false>
__global__ void __launch_bounds__(WARPS * 32)
btp_forward_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                   const __grid_constant__ CUtensorMap tm_c, const KernelParams p) {
  using LAYOUT = SmemLayout<COEF, NBOX, STAGES, WARPS, false, false, OUT_F32>;
  constexpr int TL = LAYOUT::kTL;
  constexpr int NT = LAYOUT::kTiles;
  // Loads run AHEAD chunks in front of the one being computed.  A bf16 output leaves through the
  // stage buffer itself, so a stage is reloaded only two chunks after its store was issued.
  constexpr int AHEAD = OUT_F32 ? STAGES - 1 : STAGES - 2;
  static_assert(AHEAD >= 1, "need more stages");
  static_assert(LAYOUT::kRawStages == AHEAD + 1, "a chunk's coefficients are consumed at its start");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const WarpSmem<LAYOUT, STAGES> ws = carve_smem<LAYOUT, STAGES, WARPS>(smem_raw, warp);
  const TileLane tl(lane);

  const long long nwarps = static_cast<long long>(gridDim.x) * WARPS;
  const long long wid = static_cast<long long>(blockIdx.x) * WARPS + warp;
  RunCursor cons;
  const int n = forward_work(wid, nwarps, p, cons);
  static_assert(!HANDOFF || (!OUT_F32 && !CKPT && !RAGGED), "the hand-off variant covers full chunks and 16-bit outputs");
  SeamLink seam;
  if constexpr (HANDOFF) {
    seam.set(smem_u32(smem_raw) + LAYOUT::kBytes, warp, WARPS);
    if (threadIdx.x == 0) st_shared_u32(seam.abort_word, 0u);  // visible cluster-wide after the first barrier below
  }
  // With HANDOFF every thread of the cluster passes two cluster-wide barriers: one after the barriers are
  // initialised (nobody writes into a CTA that has not set up yet), one before leaving (nobody leaves while a
  // neighbour may still write into its shared memory).  A warp without work passes both right away.
  if (n <= 0 || (smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled boxes need a 1024-byte aligned base
    if (n > 0 && lane == 0) report_error(2u, warp, 0);
    if constexpr (HANDOFF) {
      cluster_sync_all();
      cluster_sync_all();
    }
    return;
  }

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(ws.bar(s), 1);
    if constexpr (HANDOFF) {
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        mbar_init(seam.full + 8 * s, 1);
        mbar_init(seam.credit + 8 * s, 1);
      }
    }
    mbar_init_fence();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_c);
    if (!OUT_F32) prefetch_tensormap(&tm_y);
    // test hook for the give-up path: bytes that no copy will ever deliver keep this warp's first wait pending
    if (p.test_missing_tx != 0 && blockIdx.x == 0 && warp == 0) mbar_expect_tx(ws.bar(0), p.test_missing_tx);
  }
  __syncwarp();
  if constexpr (HANDOFF) cluster_sync_all();
  pdl_wait();  // nothing above touches global memory; everything below may read what the previous kernel wrote

  const int L = p.L, ncs = p.ncs;
  const float carry_scale = p.use_carry ? 1.0f : 0.0f;
  RunCursor prod = cons;
  int s_prod = 0;
  // Loads of a chunk: lanes 0 .. NBOX-1 fetch its x boxes, lane NBOX its row of coefficients (see LaneCopy).
  // A ragged last chunk is fetched whole as well: what lies beyond the sequence arrives as zeros and still
  // counts towards the barrier's byte count, so the count is a constant.
  constexpr uint32_t kChunkBytes = LAYOUT::kXBytes + LAYOUT::kRawBytes;
  // The outputs are what the next kernel of the stream reads: their lines are marked to leave L2 last.  (Measured:
  // the forward 2 % faster in its own loop, the forward+backward step 1 - 2.5 % faster, the backward 1 % slower in
  // its own loop; marking the loads, either way, was slower.)
  const uint64_t keep_out = l2_policy_evict_last();
  LaneCopy ld;
  if (lane < NBOX) ld.set(&tm_x, ws.x(0) + lane * 2048, LAYOUT::kXBytes, STAGES, 64 * lane, 16);
  else ld.set(&tm_c, ws.raw_addr(0), LAYOUT::kRawBytes, LAYOUT::kRawStages, 0, 1);
  auto issue = [&]() {  // starts the loads of the producer cursor's chunk into stage s_prod, then advances
    const uint32_t bar = ws.bar(s_prod);
    if (lane <= NBOX) {
      if (lane == 0) mbar_arrive_expect_tx(bar, kChunkBytes);
      tma_load_2d(ld.cur, ld.map, prod.cs * TL + ld.col_off, prod.bh * ld.row_mul, bar);
    }
    ld.advance();
    prod.next(ncs);
    s_prod = (s_prod + 1 == STAGES) ? 0 : s_prod + 1;
  };

  for (int k = 0; k < AHEAD && k < n; ++k) issue();

  float cg = 0.0f, cg8 = 0.0f;  // carry into the next block, channels g and g+8
  bool failed = false;
  int j = 0, s = 0;  // chunk, its stage in the x ring
  uint32_t phase = 0;
  // HANDOFF: the run in work is this warp's krun-th; its first block waits, uncorrected, for the carry from the left
  int krun = 0;
  bool owed = false;
  float f0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, f1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float2 fPa = make_float2(0.0f, 0.0f), fPb = fPa;
  unsigned short* fy = nullptr;

  for (; j < n; ++j) {
    if (j + AHEAD < n) {
      if (!OUT_F32 && lane < NBOX) bulk_wait_group_read<1>();  // this lane's store that last used that stage has drained
      if constexpr (OUT_F32 && LAYOUT::kTInPlace) {
        // the coefficient buffer about to be reloaded was last WRITTEN by this warp (the T table of the chunk
        // before); with a 16-bit output the fence in front of the chunk's store already orders that
        fence_proxy_async_smem();
        __syncwarp();
      }
      issue();
    }
    // the decision to give up is taken by the whole warp: the code below is full of warp-wide instructions
    if (!__all_sync(0xffffffffu, mbar_wait_bounded(ws.bar(s), phase, p.wait_limit_ns))) {
      failed = true;
      break;
    }
    const int nt = chunk_tiles<TL, RAGGED>(cons.cs, L);
    const int c0 = cons.cs * TL;
    // the chunk's stage in the coefficient ring, which is as long as the x ring or has two stages
    static_assert(LAYOUT::kRawStages == STAGES || LAYOUT::kRawStages == 2, "coefficient ring");
    const int rs = LAYOUT::kRawStages == STAGES ? s : (j & 1);
    // T over the raw coefficients when they are floats, else in front of P in the table area
    float* tab = LAYOUT::kTInPlace ? reinterpret_cast<float*>(ws.raw_ptr(rs)) : ws.tab_ptr(0);
    float* tabP = LAYOUT::kTInPlace ? ws.tab_ptr(0) : ws.tab_ptr(0) + TL;
    chunk_tables<COEF, TL, false, F16>(ws.raw_ptr(rs), tab, tabP, lane, carry_scale);

    if (cons.cs == 0 || !p.use_carry) {
      cg = cg8 = 0.0f;
    } else if (cons.fresh) {  // the block to the left belongs to another warp (or another run)
      if constexpr (HANDOFF) {
        cg = cg8 = 0.0f;
        owed = true;
        fy = reinterpret_cast<unsigned short*>(p.out_f32) + (static_cast<long long>(cons.bh) * 16 + tl.g) * L + c0 + 2 * tl.t;
        if (lane == 0) mbar_arrive_expect_tx(seam.full + 8 * (krun & 1), 64);
      } else {
        halo_reduce<COEF, false, false, PRECISE, F16>(p.x, p.coeff, L, cons.bh, c0 - 16, lane, cg, cg8);
      }
    }

    const float* tg = tab + tl.g;
    const float* tt = tab + 2 * tl.t;
    const float* tp = tabP + 2 * tl.t;
    const uint32_t xs = ws.x(s);
    const uint32_t ldm = xs + tl.ldm_base;
    const uint32_t stb = xs + tl.st_base;
    float* yo = nullptr;
    if constexpr (OUT_F32) {
      yo = reinterpret_cast<float*>(p.out_f32) + (static_cast<long long>(cons.bh) * 16 + tl.g) * L + c0 + 2 * tl.t;
    }
    float* ck = nullptr;
    if constexpr (CKPT) {
      ck = p.ckpt + (static_cast<long long>(cons.bh) * (L >> 4) + cons.cs * NT) * 16 + tl.g;
    }

#pragma unroll
    for (int i = 0; i < NT; ++i) {
      if (i < nt) {
        const int box = i >> 2, ib = i & 3;
        LmatFrag lf, lo;
        if constexpr (PRECISE) {
          build_lmat_split<F16>(tg, tt, 16 * i, tl, lf, lo);
        } else {
          lf = build_lmat<F16>(tg, tt, 16 * i, tl);
        }
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(ldm + box * 2048 + tl.ldm_off[ib], a0, a1, a2, a3);
        float v0[4], v1[4];
        if constexpr (PRECISE) {
          // first eight tokens: x0 . hi + x0 . lo as ONE k = 16 product, the operand x0 given twice
          Act<F16>::mma16(v0, a0, a1, a0, a1, lf.b00, lo.b00);
          Act<F16>::mma16(v1, a0, a1, a2, a3, lf.b10, lf.b11);
          Act<F16>::mma16_acc(v1, a0, a1, a2, a3, lo.b10, lo.b11);
        } else {
          Act<F16>::mma8(v0, a0, a1, lf.b00);
          Act<F16>::mma16(v1, a0, a1, a2, a3, lf.b10, lf.b11);
        }
        const float2 Pa = *reinterpret_cast<const float2*>(tp + 16 * i);
        const float2 Pb = *reinterpret_cast<const float2*>(tp + 16 * i + 8);
        // y = v + P (x) carry, a token pair per packed fp32x2 instruction (the accumulators hold tokens
        // 2t, 2t+1 of a channel side by side)
        const float2 cg2 = make_float2(cg, cg), cg82 = make_float2(cg8, cg8);
        const float2 ya = __ffma2_rn(Pa, cg2, make_float2(v0[0], v0[1]));
        const float2 yb = __ffma2_rn(Pa, cg82, make_float2(v0[2], v0[3]));
        const float2 yc = __ffma2_rn(Pb, cg2, make_float2(v1[0], v1[1]));
        const float2 yd = __ffma2_rn(Pb, cg82, make_float2(v1[2], v1[3]));
        const float y0[4] = {ya.x, ya.y, yb.x, yb.y};
        const float y1[4] = {yc.x, yc.y, yd.x, yd.y};
        if constexpr (HANDOFF) {
          if (i == 0 && cons.fresh) {  // kept for the correction at the end of the run
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              f0[e] = v0[e];
              f1[e] = v1[e];
            }
            fPa = Pa;
            fPb = Pb;
          }
        }
        if constexpr (CKPT) {
          // slot j of the checkpoint = block-local last token of block j, except the last block
          if (p.use_carry && tl.t == 3 && (cons.cs * NT + i) < (L >> 4) - 1) {
            ck[16 * i] = v1[1];
            ck[16 * i + 8] = v1[3];
          }
        }
        // carry for the next block: the UNCORRECTED last token (btp-forward.cu:297-299)
        cg = __shfl_sync(0xffffffffu, v1[1], lane | 3);
        cg8 = __shfl_sync(0xffffffffu, v1[3], lane | 3);
        if constexpr (OUT_F32) {
          const long long r8 = 8ll * L;
          *reinterpret_cast<float2*>(yo + 16 * i) = make_float2(y0[0], y0[1]);
          *reinterpret_cast<float2*>(yo + 16 * i + r8) = make_float2(y0[2], y0[3]);
          *reinterpret_cast<float2*>(yo + 16 * i + 8) = make_float2(y1[0], y1[1]);
          *reinterpret_cast<float2*>(yo + 16 * i + 8 + r8) = make_float2(y1[2], y1[3]);
        } else {
          // y replaces the consumed x block.  No warp barrier is needed in between: the block was read by ONE
          // warp-wide ldmatrix, the products that y depends on wait for that whole instruction, and the
          // shared-memory instructions of a warp execute in program order.
          const uint32_t o0 = stb + box * 2048 + tl.st_off[ib];
          const uint32_t o1 = o0 ^ 16u;
          st_shared_u32(o0, Act<F16>::pack(y0[0], y0[1]));
          st_shared_u32(o0 + 1024, Act<F16>::pack(y0[2], y0[3]));
          st_shared_u32(o1, Act<F16>::pack(y1[0], y1[1]));
          st_shared_u32(o1 + 1024, Act<F16>::pack(y1[2], y1[3]));
        }
      }
    }
    if constexpr (!OUT_F32) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane < NBOX) {  // lane b sends box b (the same lane reloads that box's buffer later)
        if (!RAGGED || c0 + 64 * lane < L) {
          tma_store_2d_hint(reinterpret_cast<uint64_t>(&tm_y), c0 + 64 * lane, cons.bh * 16, xs + lane * 2048, keep_out);
        }
        bulk_commit_group();
      }
    }
    if constexpr (HANDOFF) {
      if (cons.left == 1) {  // end of a run
        const int sl = krun & 1;
        const uint32_t use = static_cast<uint32_t>(krun >> 1);
        if (p.use_carry && cons.cs != ncs - 1) {  // the run to the right is waiting for (cg, cg8)
          bool ok = true;
          if (krun >= 2) {
            ok = mbar_wait_bounded_cluster(seam.credit + 8 * sl, (use - 1) & 1u, p.wait_limit_ns, seam.abort_word);
          }
          if (!__all_sync(0xffffffffu, ok)) {
            failed = true;
            break;
          }
          if (tl.t == 0) st_async_f32x2(seam.right_slot + 64 * sl + 8 * tl.g, cg, cg8, seam.right_full + 8 * sl);
        }
        if (owed) {
          if (!__all_sync(0xffffffffu,
                          mbar_wait_bounded_cluster(seam.full + 8 * sl, use & 1u, p.wait_limit_ns, seam.abort_word))) {
            failed = true;
            break;
          }
          float c_g, c_g8;
          asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(c_g), "=f"(c_g8) : "r"(seam.slot + 64 * sl + 8 * tl.g) : "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(seam.left_credit + 8 * sl);
          // The run's first chunk left through a TMA store with this block uncorrected.  A run has at least two
          // chunks, so when all store groups but the latest are complete, that store is.
          if (lane < NBOX) bulk_wait_group<1>();
          __syncwarp();
          const float2 cc = make_float2(c_g, c_g), cc8 = make_float2(c_g8, c_g8);
          const float2 ya = __ffma2_rn(fPa, cc, make_float2(f0[0], f0[1]));
          const float2 yb = __ffma2_rn(fPa, cc8, make_float2(f0[2], f0[3]));
          const float2 yc = __ffma2_rn(fPb, cc, make_float2(f1[0], f1[1]));
          const float2 yd = __ffma2_rn(fPb, cc8, make_float2(f1[2], f1[3]));
          const long long r8 = 8ll * L;
          *reinterpret_cast<uint32_t*>(fy) = Act<F16>::pack(ya.x, ya.y);
          *reinterpret_cast<uint32_t*>(fy + r8) = Act<F16>::pack(yb.x, yb.y);
          *reinterpret_cast<uint32_t*>(fy + 8) = Act<F16>::pack(yc.x, yc.y);
          *reinterpret_cast<uint32_t*>(fy + 8 + r8) = Act<F16>::pack(yd.x, yd.y);
          owed = false;
        }
        ++krun;
      }
    }
    cons.next(ncs);
    if (++s == STAGES) {
      s = 0;
      phase ^= 1u;
    }
  }

  if (failed) {
    if (lane == 0) report_error(1u, warp, cons.bh * ncs + cons.cs);
    if constexpr (HANDOFF) {  // nobody in the cluster needs to wait for this warp any longer
      if (lane < cluster_cta_count()) st_cluster_u32(map_to_cta(seam.abort_word, lane), 1u);
    }
    // give the loads still in flight a (bounded) chance to land before the buffers are released
    for (int k = j; k < n && k <= j + AHEAD; ++k) {
      mbar_wait_bounded(ws.bar(s), phase, p.wait_limit_ns);
      if (++s == STAGES) {
        s = 0;
        phase ^= 1u;
      }
    }
  }
  if (!OUT_F32 && lane < NBOX) bulk_wait_group<0>();
  if constexpr (HANDOFF) cluster_sync_all();
}

// =====================================================================================
// Backward
// =====================================================================================
struct TileAcc {
  float v0[4], v1[4];  // local pass   v  (channels g / g+8 x tokens 2t,2t+1 | 8+2t,9+2t)
  float g0[4], g1[4];  // gw = dy . Lmat
};

// PRECISE: the Lmat operand goes to the tensor cores as two bf16 terms (4 more products per block), which
// brings dA to the accuracy of a float32 evaluation; without it Lmat is rounded to bf16 once.
template <int COEF, bool DY_F32, bool RAGGED, bool PRECISE, int NBOX, int STAGES, int WARPS, bool F16 = false>
__global__ void __launch_bounds__(WARPS * 32)
btp_backward_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                    const __grid_constant__ CUtensorMap tm_dx, const __grid_constant__ CUtensorMap tm_c,
                    const __grid_constant__ CUtensorMap tm_da, const KernelParams p) {
  using LAYOUT = SmemLayout<COEF, NBOX, STAGES, WARPS, true, DY_F32>;
  constexpr int TL = LAYOUT::kTL;
  constexpr int NT = LAYOUT::kTiles;
  static_assert(STAGES >= 3, "the backward ring needs three stages");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const WarpSmem<LAYOUT, STAGES> ws = carve_smem<LAYOUT, STAGES, WARPS>(smem_raw, warp);
  const TileLane tl(lane);

  const long long nwarps = static_cast<long long>(gridDim.x) * WARPS;
  const long long wid = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const WarpWork work(wid, nwarps, p.total_chunks, p.ncs, p.interleave != 0, true);
  const int n = work.n;
  if (n <= 0) return;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled boxes need a 1024-byte aligned base
    if (lane == 0) report_error(2u, warp, 0);
    return;
  }

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(ws.bar(s), 1);
    mbar_init_fence();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_dy);
    prefetch_tensormap(&tm_dx);
    prefetch_tensormap(&tm_c);
    prefetch_tensormap(&tm_da);
    if (p.test_missing_tx != 0 && blockIdx.x == 0 && warp == 0) mbar_expect_tx(ws.bar(0), p.test_missing_tx);  // see forward
  }
  __syncwarp();
  pdl_wait();  // nothing above touches global memory

  const int L = p.L, ncs = p.ncs;
  const float carry_scale = p.use_carry ? 1.0f : 0.0f;
  ChunkCursor prod(work.bh, work.cs, work.step), cons(work.bh, work.cs, work.step);
  int s_prod = 0, issued = 0;
  // Loads of a chunk (see LaneCopy): lanes 0 .. NBOX-1 its x boxes, the next NDY lanes its dy boxes (a float dy
  // takes two 32-token boxes per 64 tokens), the lane after them its row of coefficients.  The dy ring is one
  // stage shorter than the x ring; every lane steps through its own ring.  Ragged chunks are fetched whole.
  constexpr int NDY = DY_F32 ? 2 * NBOX : NBOX;
  constexpr int kLoadLanes = NBOX + NDY + 1;
  constexpr uint32_t kChunkBytes = LAYOUT::kXBytes + LAYOUT::kDyBytes + LAYOUT::kRawBytes;
  LaneCopy ld;
  if (lane < NBOX) ld.set(&tm_x, ws.x(0) + lane * 2048, LAYOUT::kXBytes, STAGES, 64 * lane, 16);
  else if (lane < NBOX + NDY) ld.set(&tm_dy, ws.dy(0) + (lane - NBOX) * 2048, LAYOUT::kDyBytes, STAGES - 1,
                                     (DY_F32 ? 32 : 64) * (lane - NBOX), 16);
  else ld.set(&tm_c, ws.raw_addr(0), LAYOUT::kRawBytes, STAGES, 0, 1);
  const uint64_t keep_out = l2_policy_evict_last();  // as in the forward: the outputs leave L2 last
  // Stores of a chunk: lanes 0 .. NBOX-1 its dx boxes (out of the x buffers), lane NBOX its row of dA.
  LaneCopy st;
  if (lane < NBOX) st.set(&tm_dx, ws.x(0) + lane * 2048, LAYOUT::kXBytes, STAGES, 64 * lane, 16);
  else st.set(&tm_da, ws.da_addr(0), LAYOUT::kDaBytes, STAGES, 0, 1);
  auto issue = [&]() {
    const uint32_t bar = ws.bar(s_prod);
    if (lane < kLoadLanes) {
      if (lane == 0) mbar_arrive_expect_tx(bar, kChunkBytes);
      tma_load_2d(ld.cur, ld.map, prod.cs * TL + ld.col_off, prod.bh * ld.row_mul, bar);
    }
    ld.advance();
    prod.next(ncs);
    s_prod = (s_prod + 1 == STAGES) ? 0 : s_prod + 1;
    ++issued;
  };

  // Chunk j's outputs leave one block into chunk j+1 (its last block needs the gradient that
  // arrives from the right).  The x buffer of chunk j is reloaded at the end of chunk j+1, when that
  // store has certainly drained; the dy buffer of chunk j is free once chunk j's products are done.
  // Loads therefore run a whole chunk ahead of the one in work, and STAGES-1 dy buffers are enough.
  while (issued < STAGES - 1 && issued < n) issue();

  // ---- front half of a block: Lmat fragments and the four tensor-core products
  auto front = [&](const float* tab, const float* tg, const float* tt, uint32_t ldm_x, uint32_t dy_s, int i,
                   TileAcc& acc, float& dc_g, float& dc_g8) {  // dy_s: the chunk's dy buffer
    const int box = i >> 2, ib = i & 3;
    LmatFrag lf, lo;
    if constexpr (PRECISE) {
      build_lmat_split<F16>(tg, tt, 16 * i, tl, lf, lo);
    } else {
      lf = build_lmat<F16>(tg, tt, 16 * i, tl);
    }
    // dy . Lmat needs the transposed 8x8 blocks as B operand (k = r, n = c)
    const uint32_t g00 = movmatrix_trans(lf.b00);
    const uint32_t g10 = movmatrix_trans(lf.b10);
    const uint32_t g11 = movmatrix_trans(lf.b11);
    uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
    uint32_t l0 = 0, l1 = 0, l2 = 0, l3 = 0;  // second bf16 term of a float32 dy
    ldmatrix_x4(ldm_x + box * 2048 + tl.ldm_off[ib], a0, a1, a2, a3);
    if constexpr (DY_F32) {
      // [16][32] float boxes, 128-byte swizzle: block i sits in box i/2 at byte offset (i&1)*64 of each row
      const uint32_t bb = dy_s + (i >> 1) * 2048 + tl.g * 128;
      const uint32_t c_lo = ((i & 1) * 4 + (tl.t >> 1)), c_hi = c_lo + 2;
      const uint32_t in = (tl.t & 1) * 8;
      auto lds = [&](uint32_t addr) {
        float2 r;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "r"(addr));
        return r;
      };
      // A float32 dy goes to the tensor cores as two bf16 terms as well (hi + lo), so that dA keeps float32
      // accuracy for float32 upstream gradients (the op's default output type makes them float32).
      auto split = [&](const float2 f, uint32_t& hi, uint32_t& lo) {
        hi = Act<F16>::pack(f.x, f.y);
        if constexpr (PRECISE) lo = Act<F16>::pack(f.x - Act<F16>::lo(hi), f.y - Act<F16>::hi(hi));
      };
      split(lds(bb + ((c_lo ^ tl.g) << 4) + in), e0, l0);
      split(lds(bb + 1024 + ((c_lo ^ tl.g) << 4) + in), e1, l1);
      split(lds(bb + ((c_hi ^ tl.g) << 4) + in), e2, l2);
      split(lds(bb + 1024 + ((c_hi ^ tl.g) << 4) + in), e3, l3);
    } else {
      ldmatrix_x4(dy_s + tl.ldm_base + box * 2048 + tl.ldm_off[ib], e0, e1, e2, e3);
    }
    using A = Act<F16>;
    if constexpr (PRECISE) {
      // The two 8-token products (x0 . L00 and dy1 . L11) take their hi and lo terms in ONE k = 16 instruction
      // each, with the left operand given twice; the two 16-token products take two instructions.
      A::mma16(acc.v0, a0, a1, a0, a1, lf.b00, lo.b00);
      A::mma16(acc.v1, a0, a1, a2, a3, lf.b10, lf.b11);
      A::mma16_acc(acc.v1, a0, a1, a2, a3, lo.b10, lo.b11);
      A::mma16(acc.g0, e0, e1, e2, e3, g00, g10);
      A::mma16_acc(acc.g0, e0, e1, e2, e3, movmatrix_trans(lo.b00), movmatrix_trans(lo.b10));
      A::mma16(acc.g1, e2, e3, e2, e3, g11, movmatrix_trans(lo.b11));
      if constexpr (DY_F32) {  // dy_lo . Lmat_hi (the lo . lo term is below float32 resolution)
        A::mma16_acc(acc.g0, l0, l1, l2, l3, g00, g10);
        A::mma8_acc(acc.g1, l2, l3, g11);
      }
    } else {
      A::mma8(acc.v0, a0, a1, lf.b00);
      A::mma16(acc.v1, a0, a1, a2, a3, lf.b10, lf.b11);
      A::mma16(acc.g0, e0, e1, e2, e3, g00, g10);
      A::mma8(acc.g1, e2, e3, g11);
    }
    // gradient this block sends to its left neighbour: P[0] * gw[:,0]   (P[0] = Pshift[1])
    const float a_first = tab[TL + 16 * i + 1];
    dc_g = a_first * __shfl_sync(0xffffffffu, acc.g0[0], lane & ~3);
    dc_g8 = a_first * __shfl_sync(0xffffffffu, acc.g0[2], lane & ~3);
  };

  // ---- back half of a block: everything that needs the gradient arriving from the right.
  // tt_i = &T[16 i + 2t] of the block's chunk, da_i = &dA_stage[16 i], o0 = dx store address.
  auto back = [&](const TileAcc& acc, const float* tt_i, float* da_i, uint32_t o0, float cg, float cg8, float dc_g,
                  float dc_g8) {
    const float2 Sa = *reinterpret_cast<const float2*>(tt_i + TL);          // P[2t-1], P[2t]
    const float2 Sb = *reinterpret_cast<const float2*>(tt_i + TL + 8);      // P[2t+7], P[2t+8]
    const float2 La = *reinterpret_cast<const float2*>(tt_i + 2 * TL);      // Lmat[15, 2t], Lmat[15, 2t+1]
    const float2 Lb = *reinterpret_cast<const float2*>(tt_i + 2 * TL + 8);  // Lmat[15, 2t+8], Lmat[15, 2t+9]
    // Packed fp32x2 arithmetic (one instruction for a token pair): the accumulator registers already hold
    // tokens (2t, 2t+1) of a channel side by side.
    const float2 dcg = make_float2(dc_g, dc_g), dcg8 = make_float2(dc_g8, dc_g8);
    const float2 g0a = make_float2(acc.g0[0], acc.g0[1]), g0b = make_float2(acc.g0[2], acc.g0[3]);
    const float2 g1a = make_float2(acc.g1[0], acc.g1[1]), g1b = make_float2(acc.g1[2], acc.g1[3]);
    const float2 dxa = __ffma2_rn(La, dcg, g0a);   // channel g,   tokens 2t, 2t+1
    const float2 dxb = __ffma2_rn(La, dcg8, g0b);  // channel g+8
    const float2 dxc = __ffma2_rn(Lb, dcg, g1a);   // channel g,   tokens 8+2t, 9+2t
    const float2 dxd = __ffma2_rn(Lb, dcg8, g1b);  // channel g+8
    const float dx0[4] = {dxa.x, dxa.y, dxb.x, dxb.y};
    const float dx1[4] = {dxc.x, dxc.y, dxd.x, dxd.y};
    // v shifted right by one token
    const int src = (lane & ~3) | ((lane + 3) & 3);
    const float A_g = __shfl_sync(0xffffffffu, acc.v0[1], src);
    const float A_g8 = __shfl_sync(0xffffffffu, acc.v0[3], src);
    const float B_g = __shfl_sync(0xffffffffu, acc.v1[1], src);
    const float B_g8 = __shfl_sync(0xffffffffu, acc.v1[3], src);
    const float2 vpa = make_float2(tl.t ? A_g : 0.0f, acc.v0[0]), vpb = make_float2(tl.t ? A_g8 : 0.0f, acc.v0[2]);
    const float2 vpc = make_float2(tl.t ? B_g : A_g, acc.v1[0]), vpd = make_float2(tl.t ? B_g8 : A_g8, acc.v1[2]);
    const float2 cg2 = make_float2(cg, cg), cg82 = make_float2(cg8, cg8);
    float2 m01 = __ffma2_rn(vpa, dxa, __fmul2_rn(vpb, dxb));
    float2 m23 = __ffma2_rn(vpc, dxc, __fmul2_rn(vpd, dxd));
    m01 = __ffma2_rn(Sa, __ffma2_rn(g0a, cg2, __fmul2_rn(g0b, cg82)), m01);
    m23 = __ffma2_rn(Sb, __ffma2_rn(g1a, cg2, __fmul2_rn(g1b, cg82)), m23);
    // sum over the 16 channels: channel pairs are in-thread, the 8 groups g are folded by a
    // transposing butterfly (each step halves the number of tokens a lane keeps)
    const bool b0 = (tl.g & 1) != 0, b1 = (tl.g & 2) != 0;
    const float2 keepv = b0 ? m23 : m01, sendv = b0 ? m01 : m23;
    const float2 r01 = __fadd2_rn(keepv, make_float2(__shfl_xor_sync(0xffffffffu, sendv.x, 4),
                                                     __shfl_xor_sync(0xffffffffu, sendv.y, 4)));
    const float r0 = r01.x, r1 = r01.y;
    const float keep = b1 ? r1 : r0, send = b1 ? r0 : r1;
    float r = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    r += __shfl_xor_sync(0xffffffffu, r, 16);
    if (lane < 16) {
      // token kept by this lane: [2t, 2t+1, 2t+8, 2t+9][2*b0 + b1]
      const int tok = 2 * tl.t + (b1 ? 1 : 0) + (b0 ? 8 : 0);
      if constexpr (COEF == kCoefF32Log) {
        // gradient w.r.t. the log coefficient: dA * a,  a_tok = P[tok] / P[tok-1] = 2^(T_tok - T_{tok-1})
        const float* Tt = tt_i - 2 * tl.t;
        const float Tprev = tok ? Tt[tok - 1] : 0.0f;
        r *= ex2(Tt[tok] - Tprev);
      }
      da_i[tok] = r;
    }
    // dx replaces the consumed x block in shared memory
    const uint32_t o1 = o0 ^ 16u;
    st_shared_u32(o0, Act<F16>::pack(dx0[0], dx0[1]));
    st_shared_u32(o0 + 1024, Act<F16>::pack(dx0[2], dx0[3]));
    st_shared_u32(o1, Act<F16>::pack(dx1[0], dx1[1]));
    st_shared_u32(o1 + 1024, Act<F16>::pack(dx1[2], dx1[3]));
  };

  // pending block = last block of the previous chunk; its accumulators live in slot B
  TileAcc accA, accB;
  bool have = false, failed = false;
  bool p_seq_end = false;
  const float* p_tt = nullptr;
  float* p_da = nullptr;
  uint32_t p_o0 = 0;
  float p_cg = 0.0f, p_cg8 = 0.0f;
  int p_stage = 0, p_bh = 0, p_c0 = 0, p_nt = 0;
  float vl_g = 0.0f, vl_g8 = 0.0f;  // uncorrected last token of the most recent block

  auto flush = [&]() {  // the pending block's chunk is complete: send dx and dA on their way
    fence_proxy_async_smem();
    __syncwarp();
    if (lane <= NBOX) {
      // a ragged chunk is stored whole too: the copy clips what lies beyond the sequence
      if (!RAGGED || p_c0 + st.col_off < L) {
        tma_store_2d_hint(st.map, p_c0 + st.col_off, p_bh * st.row_mul, st.at(p_stage), keep_out);
      }
      bulk_commit_group();
    }
  };
  // The loads of chunk j+1 start as soon as chunk j-1's last products are done: its dy buffer is dead then, and the
  // x buffer it goes into last held chunk j-2, whose store left three blocks ago and has long been read out.
  auto issue_next = [&]() {
    if (issued < n) {
      if (lane <= NBOX) bulk_wait_group_read<0>();
      issue();
    }
  };

  int j = 0, s = 0, d = 0, tset = 0;
  uint32_t phase = 0;
  for (; j < n; ++j) {
    if (!__all_sync(0xffffffffu, mbar_wait_bounded(ws.bar(s), phase, p.wait_limit_ns))) {  // warp-uniform, as in forward
      failed = true;
      break;
    }
    const int nt = chunk_tiles<TL, RAGGED>(cons.cs, L);
    const int c0 = cons.cs * TL;
    float* tab = ws.tab_ptr(tset);
    chunk_tables<COEF, TL, true, F16>(ws.raw_ptr(s), tab, tab + TL, lane, carry_scale);
    if (j == 0 && cons.cs != 0 && p.use_carry) {
      halo_reduce<COEF, false, false, PRECISE, F16>(p.x, p.coeff, L, cons.bh, c0 - 16, lane, vl_g, vl_g8);
    }
    const float* tg = tab + tl.g;
    const float* tt = tab + 2 * tl.t;
    float* da = ws.da_ptr(s);
    const uint32_t xs = ws.x(s);
    const uint32_t dys = ws.dy(d);
    const uint32_t ldm = xs + tl.ldm_base;
    const uint32_t stb = xs + tl.st_base;
    const bool seq_first = (cons.cs == 0);

#pragma unroll
    for (int i = 0; i < NT; ++i) {
      if (i < nt) {
        TileAcc& cur = (i & 1) ? accB : accA;         // block i
        const TileAcc& prev = (i & 1) ? accA : accB;  // block i-1 (slot B holds the pending one when i == 0)
        float dc_g, dc_g8;
        front(tab, tg, tt, ldm, dys, i, cur, dc_g, dc_g8);
        const float ncg = (i == 0 && seq_first) ? 0.0f : vl_g;  // carry into block i
        const float ncg8 = (i == 0 && seq_first) ? 0.0f : vl_g8;
        if (i == 0) {
          if (have) {
            back(prev, p_tt, p_da, p_o0, p_cg, p_cg8, p_seq_end ? 0.0f : dc_g, p_seq_end ? 0.0f : dc_g8);
            flush();
          }
        } else {
          const int pi = i - 1;
          back(prev, tt + 16 * pi, da + 16 * pi, stb + (pi >> 2) * 2048 + tl.st_off[pi & 3], p_cg, p_cg8, dc_g, dc_g8);
        }
        p_cg = ncg;
        p_cg8 = ncg8;
        vl_g = __shfl_sync(0xffffffffu, cur.v1[1], lane | 3);
        vl_g8 = __shfl_sync(0xffffffffu, cur.v1[3], lane | 3);
      }
    }
    // the chunk's last block becomes the pending one (slot B)
    if ((nt & 1) != 0) accB = accA;
    have = true;
    p_seq_end = (cons.cs == ncs - 1);
    p_tt = tt + 16 * (nt - 1);
    p_da = da + 16 * (nt - 1);
    p_o0 = stb + ((nt - 1) >> 2) * 2048 + (((2u * ((nt - 1) & 3)) ^ static_cast<uint32_t>(tl.g)) << 4);
    p_stage = s;
    p_bh = cons.bh;
    p_c0 = c0;
    p_nt = nt;
    issue_next();
    cons.next(ncs);
    tset ^= 1;
    if (++d == STAGES - 1) d = 0;
    if (++s == STAGES) {
      s = 0;
      phase ^= 1u;
    }
  }

  if (!failed && have) {
    float dc_g = 0.0f, dc_g8 = 0.0f;
    if (!p_seq_end && p.use_carry) {
      // the block to the right belongs to another warp: recompute what it sends
      halo_reduce<COEF, DY_F32, true, PRECISE, F16>(p.dy, p.coeff, L, p_bh, p_c0 + 16 * p_nt, lane, dc_g, dc_g8);
    }
    back(accB, p_tt, p_da, p_o0, p_cg, p_cg8, dc_g, dc_g8);
    flush();
  }
  if (failed) {
    if (lane == 0) report_error(1u, warp, cons.bh * ncs + cons.cs);
    for (int k = j; k < issued; ++k) {
      mbar_wait_bounded(ws.bar(s), phase, p.wait_limit_ns);
      if (++s == STAGES) {
        s = 0;
        phase ^= 1u;
      }
    }
  }
  if (lane <= NBOX) bulk_wait_group<0>();
}

}  // namespace btp
