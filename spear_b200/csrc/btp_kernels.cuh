// BTP forward and backward kernels for sm_100a.
//
// What is computed (per (b,h) sequence, 16 channels, blocks of 16 tokens; semantics of
// spear/ops/btp/reference.py:105-139 and csrc/btp/btp-forward.cu:85-457,
// csrc/btp/btp-backwards.cu:165-808):
//   T_r       = sum_{j<=r} log2 a_j                      (inclusive, per block)
//   Lmat[r,c] = 2^(T_r - T_c) for c <= r, else 0         P[r] = 2^(T_r)
//   v_i       = x_i . Lmat^T                             (local pass, tensor cores)
//   y_i       = v_i + P (x) carry_i,   carry_i = v_{i-1}[:,15]   (ONE hop, never the corrected value)
//   gw_i      = dy_i . Lmat,  dCarry_i = 2^(T_0) gw_i[:,0]
//   dx_i[:,c] = gw_i[:,c] + Lmat[15,c] dCarry_{i+1}
//   dA_i[t]   = sum_ch v_i[ch,t-1] dx_i[ch,t] + P[t-1] sum_ch gw_i[ch,t] carry_i[ch]
//               (v[:, -1] = 0, P[-1] = 1; no division by a anywhere)
//
// How it is mapped to the machine:
//   * Work unit = a chunk of TL = 64*NBOX tokens of one sequence: x as NBOX TMA boxes of
//     [16 channels x 64 tokens] bf16 (128-byte swizzle), the coefficients as one bulk copy.
//   * Every WARP owns a private ring of STAGES chunk buffers with its own mbarriers and walks a
//     contiguous range of chunks.  No block-wide or grid-wide synchronisation exists, so no warp
//     ever waits for another warp; the only waits are on the warp's own TMA loads (bounded).
//   * The carry stays in registers while a warp walks along a sequence.  Where a warp's range
//     starts (ends) inside a sequence the neighbouring block is re-read from global memory
//     (16x16 values, a "halo") and its carry (dCarry) recomputed, so no seam ever drops a carry.
//   * Outputs in bf16 are written over the consumed input tile in shared memory and leave with a
//     TMA store; fp32 outputs are stored straight from the accumulator fragments (32-byte runs).
#pragma once

#include "btp_ptx.cuh"

namespace btp {

constexpr int kCoefBf16 = 0;    // linear coefficient, bf16
constexpr int kCoefF32 = 1;     // linear coefficient, float
constexpr int kCoefF32Log = 2;  // natural-log coefficient, float

constexpr float kLog2E = 1.4426950408889634f;
constexpr float kZeroLog2 = -200.0f;  // stands in for log2(0): 2^-200 flushes to zero, sums stay finite
constexpr float kTinyCoeff = 1e-9f;   // coefficients at or below this count as zero (btp-forward.cu:179)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // bounded waits give up after 2 s

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

// Shared-memory carve-up of one CTA.  Every warp owns STAGES stages.
template <int NBOX, int STAGES, int WARPS, bool BWD, bool DY_F32>
struct SmemLayout {
  static constexpr int kTL = 64 * NBOX;                 // tokens per chunk
  static constexpr int kTiles = kTL / 16;               // 16-token blocks per chunk
  static constexpr int kXBytes = NBOX * 2048;           // [16][64] bf16 per box
  static constexpr int kDyBytes = BWD ? (DY_F32 ? NBOX * 4096 : NBOX * 2048) : 0;
  static constexpr int kBigPerStage = kXBytes + kDyBytes;  // multiple of 1024 (swizzle atom)
  static constexpr int kTBytes = kTL * 4;               // coefficient landing zone, then T (float)
  static constexpr int kDaBytes = BWD ? kTL * 4 : 0;
  static constexpr int kSmallPerStage = kTBytes + kDaBytes;
  static constexpr int kBigTotal = WARPS * STAGES * kBigPerStage;
  static constexpr int kSmallTotal = WARPS * STAGES * kSmallPerStage;
  static constexpr int kBarTotal = WARPS * STAGES * 8;
  static constexpr int kBytes = kBigTotal + kSmallTotal + kBarTotal + 1024;  // + slack to align the base
};

// Per-warp view of its stages.
template <class LAYOUT, int STAGES>
struct WarpSmem {
  uint32_t big;    // shared-space address of stage 0 of the tile buffers
  uint32_t small;  // ... of the T / dA buffers
  uint32_t bars;   // ... of the mbarriers
  unsigned char* small_ptr;  // generic pointer to `small`
  __device__ __forceinline__ uint32_t x(int s) const { return big + s * LAYOUT::kBigPerStage; }
  __device__ __forceinline__ uint32_t dy(int s) const { return x(s) + LAYOUT::kXBytes; }
  __device__ __forceinline__ uint32_t t_addr(int s) const { return small + s * LAYOUT::kSmallPerStage; }
  __device__ __forceinline__ float* t_ptr(int s) const {
    return reinterpret_cast<float*>(small_ptr + s * LAYOUT::kSmallPerStage);
  }
  __device__ __forceinline__ uint32_t da_addr(int s) const { return t_addr(s) + LAYOUT::kTBytes; }
  __device__ __forceinline__ float* da_ptr(int s) const {
    return reinterpret_cast<float*>(small_ptr + s * LAYOUT::kSmallPerStage + LAYOUT::kTBytes);
  }
  __device__ __forceinline__ uint32_t bar(int s) const { return bars + s * 8; }
};

template <class LAYOUT, int STAGES, int WARPS>
__device__ __forceinline__ WarpSmem<LAYOUT, STAGES> carve_smem(unsigned char* raw, int warp) {
  const uint32_t base = smem_u32(raw);
  const uint32_t pad = (1024u - (base & 1023u)) & 1023u;
  WarpSmem<LAYOUT, STAGES> w;
  w.big = base + pad + warp * STAGES * LAYOUT::kBigPerStage;
  w.small = base + pad + LAYOUT::kBigTotal + warp * STAGES * LAYOUT::kSmallPerStage;
  w.small_ptr = raw + pad + LAYOUT::kBigTotal + warp * STAGES * LAYOUT::kSmallPerStage;
  w.bars = base + pad + LAYOUT::kBigTotal + LAYOUT::kSmallTotal + warp * STAGES * 8;
  return w;
}

struct ChunkPos {
  int bh;  // sequence index
  int cs;  // chunk index inside the sequence
  int c0;  // first token
  int nt;  // 16-token blocks in this chunk (ragged last chunk: fewer)
};

template <int TL>
__device__ __forceinline__ ChunkPos chunk_pos(int id, int ncs, int L) {
  ChunkPos p;
  p.bh = id / ncs;
  p.cs = id - p.bh * ncs;
  p.c0 = p.cs * TL;
  const int left = (L - p.c0) >> 4;
  p.nt = left < TL / 16 ? left : TL / 16;
  return p;
}

// Turns the raw coefficients of a chunk (already in shared memory at `tbuf`) into per-block
// inclusive prefix sums of log2 a, in place.  Lane l owns tokens 4l..4l+3; four lanes = one block.
template <int COEF, int TL>
__device__ __forceinline__ void coeff_to_prefix(float* tbuf, int lane) {
  constexpr int kLanes = TL / 4;
  const int l = (kLanes == 32) ? lane : (lane & (kLanes - 1));
  float v0, v1, v2, v3;
  if constexpr (COEF == kCoefBf16) {
    const uint2 raw = reinterpret_cast<const uint2*>(tbuf)[l];
    v0 = bf16_lo(raw.x); v1 = bf16_hi(raw.x); v2 = bf16_lo(raw.y); v3 = bf16_hi(raw.y);
  } else {
    const float4 raw = reinterpret_cast<const float4*>(tbuf)[l];
    v0 = raw.x; v1 = raw.y; v2 = raw.z; v3 = raw.w;
  }
  const float s0 = coef_log2<COEF>(v0);
  const float s1 = s0 + coef_log2<COEF>(v1);
  const float s2 = s1 + coef_log2<COEF>(v2);
  const float s3 = s2 + coef_log2<COEF>(v3);
  const float u1 = __shfl_up_sync(0xffffffffu, s3, 1, 4);
  const float u2 = __shfl_up_sync(0xffffffffu, s3, 2, 4);
  const float u3 = __shfl_up_sync(0xffffffffu, s3, 3, 4);
  const int q = lane & 3;
  float e = 0.0f;
  if (q >= 1) e += u1;
  if (q >= 2) e += u2;
  if (q >= 3) e += u3;
  __syncwarp();  // every lane has read its raw coefficients
  if (kLanes == 32 || lane < kLanes) {
    reinterpret_cast<float4*>(tbuf)[l] = make_float4(s0 + e, s1 + e, s2 + e, s3 + e);
  }
  __syncwarp();
}

// Halo: a 16x16 block that belongs to a neighbouring warp's range is read straight from global
// memory and reduced to the 16 numbers the seam needs.
//   LEFT  (RIGHT == false): carry  = sum_c  x[ch,c] * bf16(2^(T_15 - T_c))             (= v[:,15])
//   RIGHT (RIGHT == true) : dCarry = 2^(T_0) * sum_r dy[ch,r] * bf16(2^(T_r - T_0))
// The weights are rounded to bf16 exactly like the Lmat operand of the tensor-core path.
// Returns the values for channels g and g+8 (g = lane >> 2), identical in the 4 lanes of a group.
template <int COEF, bool TILE_F32, bool RIGHT>
__device__ __forceinline__ void halo_reduce(const void* tile_base, const void* coeff_base, int L, long long bh,
                                            int tok0, int lane, float& out_g, float& out_g8) {
  const int g = lane >> 2, t = lane & 3;
  float a;
  if constexpr (COEF == kCoefBf16) {
    a = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(coeff_base)[bh * L + tok0 + (lane & 15)]);
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
    w[j] = round_bf16(ex2(RIGHT ? (Tj - Tref) : (Tref - Tj)));
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
    // the tensor-core path feeds dy rounded to bf16
    e[0][0] = round_bf16(a0.x); e[0][1] = round_bf16(a0.y); e[0][2] = round_bf16(a1.x); e[0][3] = round_bf16(a1.y);
    e[1][0] = round_bf16(b0.x); e[1][1] = round_bf16(b0.y); e[1][2] = round_bf16(b1.x); e[1][3] = round_bf16(b1.y);
  } else {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(tile_base);
    const uint32_t a0 = *reinterpret_cast<const uint32_t*>(p + row_g + 2 * t);
    const uint32_t a1 = *reinterpret_cast<const uint32_t*>(p + row_g + 8 + 2 * t);
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(p + row_g8 + 2 * t);
    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(p + row_g8 + 8 + 2 * t);
    e[0][0] = bf16_lo(a0); e[0][1] = bf16_hi(a0); e[0][2] = bf16_lo(a1); e[0][3] = bf16_hi(a1);
    e[1][0] = bf16_lo(b0); e[1][1] = bf16_hi(b0); e[1][2] = bf16_lo(b1); e[1][3] = bf16_hi(b1);
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

// Lane-constant indexing of a 16x16 bf16 tile inside a 128-byte-swizzled [16][64] box.
struct TileLane {
  int g, t;
  uint32_t ldm_row_off;  // ldmatrix: byte offset of this lane's row
  uint32_t ldm_rx;       // ldmatrix: row & 7 (swizzle key)
  uint32_t ldm_hsel;     // ldmatrix: which 8-token half this lane addresses
  bool m0, m1;           // 2t <= g, 2t+1 <= g  (causal mask of the fragment elements)
  __device__ __forceinline__ explicit TileLane(int lane) {
    g = lane >> 2;
    t = lane & 3;
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    ldm_row_off = row * 128;
    ldm_rx = row & 7;
    ldm_hsel = lane >> 4;
    m0 = (2 * t) <= g;
    m1 = (2 * t + 1) <= g;
  }
  // address for ldmatrix.x4 of block i (0..3 inside its box) -> A fragment (channels x tokens)
  __device__ __forceinline__ uint32_t ldm_addr(uint32_t box_base, int ib) const {
    return box_base + ldm_row_off + (((ib * 2 + ldm_hsel) ^ ldm_rx) << 4);
  }
  // address of the 4 bytes (channel g, tokens 2t..2t+1) of token-half `half` of block ib; channel g+8 is +1024
  __device__ __forceinline__ uint32_t frag_addr(uint32_t box_base, int ib, int half) const {
    return box_base + g * 128 + (((ib * 2 + half) ^ g) << 4) + t * 4;
  }
};

// Lmat fragments of one block for the local pass v = x . Lmat^T  (B operand: k = c, n = r).
struct LmatFrag {
  uint32_t b00;  // rows 0..7  x cols 0..7
  uint32_t b10;  // rows 8..15 x cols 0..7
  uint32_t b11;  // rows 8..15 x cols 8..15
};

__device__ __forceinline__ LmatFrag build_lmat(const float* Tt, const TileLane& tl, float2& Ta, float2& Tb) {
  const float Tg = Tt[tl.g];
  const float Tg8 = Tt[tl.g + 8];
  Ta = *reinterpret_cast<const float2*>(Tt + 2 * tl.t);
  Tb = *reinterpret_cast<const float2*>(Tt + 8 + 2 * tl.t);
  const float e0 = tl.m0 ? ex2(Tg - Ta.x) : 0.0f;
  const float e1 = tl.m1 ? ex2(Tg - Ta.y) : 0.0f;
  const float e2 = ex2(Tg8 - Ta.x);
  const float e3 = ex2(Tg8 - Ta.y);
  const float e4 = tl.m0 ? ex2(Tg8 - Tb.x) : 0.0f;
  const float e5 = tl.m1 ? ex2(Tg8 - Tb.y) : 0.0f;
  LmatFrag f;
  f.b00 = pack_bf16x2(e0, e1);
  f.b10 = pack_bf16x2(e2, e3);
  f.b11 = pack_bf16x2(e4, e5);
  return f;
}

__device__ __forceinline__ void report_timeout(int warp, int chunk) {
  if (atomicCAS(&g_btp_device_error[0], 0u, 1u) == 0u) {
    g_btp_device_error[1] = blockIdx.x;
    g_btp_device_error[2] = warp;
    g_btp_device_error[3] = chunk;
  }
}

// =====================================================================================
// Forward
// =====================================================================================
template <int COEF, bool OUT_F32, bool CKPT, int NBOX, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
btp_forward_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                   const KernelParams p) {
  using LAYOUT = SmemLayout<NBOX, STAGES, WARPS, false, false>;
  constexpr int TL = LAYOUT::kTL;
  constexpr int kEsz = CoefTraits<COEF>::kBytes;
  // Loads run AHEAD chunks in front of the one being computed.  A bf16 output leaves through the
  // stage buffer itself, so a stage is reloaded only two chunks after its store was issued.
  constexpr int AHEAD = OUT_F32 ? STAGES - 1 : STAGES - 2;
  static_assert(AHEAD >= 1, "need more stages");

  extern __shared__ unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const WarpSmem<LAYOUT, STAGES> ws = carve_smem<LAYOUT, STAGES, WARPS>(smem_raw, warp);
  const TileLane tl(lane);

  // contiguous range of chunks for this warp
  const long long nwarps = static_cast<long long>(gridDim.x) * WARPS;
  const long long wid = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const int cb = static_cast<int>((wid * p.total_chunks) / nwarps);
  const int ce = static_cast<int>(((wid + 1) * p.total_chunks) / nwarps);
  const int n = ce - cb;
  if (n <= 0) return;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(ws.bar(s), 1);
    mbar_init_fence();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_x);
    if (!OUT_F32) prefetch_tensormap(&tm_y);
  }
  __syncwarp();

  auto issue = [&](int j) {  // lane 0: start the loads of local chunk j into its stage
    const ChunkPos c = chunk_pos<TL>(cb + j, p.ncs, p.L);
    const int s = j % STAGES;
    const int nbox = (c.nt + 3) >> 2;
    const uint32_t cbytes = c.nt * 16 * kEsz;
    mbar_arrive_expect_tx(ws.bar(s), nbox * 2048 + cbytes);
    for (int b = 0; b < nbox; ++b) tma_load_2d(ws.x(s) + b * 2048, &tm_x, c.c0 + 64 * b, c.bh * 16, ws.bar(s));
    bulk_load(ws.t_addr(s), reinterpret_cast<const char*>(p.coeff) + (static_cast<long long>(c.bh) * p.L + c.c0) * kEsz,
              cbytes, ws.bar(s));
  };

  if (lane == 0) {
    for (int j = 0; j < AHEAD && j < n; ++j) issue(j);
  }

  float cg = 0.0f, cg8 = 0.0f;  // carry into the next block, channels g and g+8
  bool failed = false;
  int pending_from = 0;  // first local chunk whose load may still be in flight (for the failure path)

  for (int j = 0; j < n; ++j) {
    const int s = j % STAGES;
    const ChunkPos c = chunk_pos<TL>(cb + j, p.ncs, p.L);
    if (lane == 0 && j + AHEAD < n) {
      if (!OUT_F32) bulk_wait_group_read<1>();  // the store that last used that stage has drained
      issue(j + AHEAD);
    }
    pending_from = j;
    if (!mbar_wait_bounded(ws.bar(s), (j / STAGES) & 1, kWaitLimitNs)) {
      failed = true;
      break;
    }
    pending_from = j + 1;
    float* T = ws.t_ptr(s);
    coeff_to_prefix<COEF, TL>(T, lane);

    if (c.cs == 0 || !p.use_carry) {
      cg = cg8 = 0.0f;
    } else if (j == 0) {
      halo_reduce<COEF, false, false>(p.x, p.coeff, p.L, c.bh, c.c0 - 16, lane, cg, cg8);
    }

    for (int i = 0; i < c.nt; ++i) {
      const int box = i >> 2, ib = i & 3;
      const uint32_t box_base = ws.x(s) + box * 2048;
      float2 Ta, Tb;
      const LmatFrag lf = build_lmat(T + 16 * i, tl, Ta, Tb);
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(tl.ldm_addr(box_base, ib), a0, a1, a2, a3);
      float v0[4], v1[4];
      mma_1688(v0, a0, a1, lf.b00);
      mma_16816(v1, a0, a1, a2, a3, lf.b10, lf.b11);
      const float p0 = ex2(Ta.x), p1 = ex2(Ta.y), p2 = ex2(Tb.x), p3 = ex2(Tb.y);
      float y0[4], y1[4];
      y0[0] = fmaf(p0, cg, v0[0]);  y0[1] = fmaf(p1, cg, v0[1]);
      y0[2] = fmaf(p0, cg8, v0[2]); y0[3] = fmaf(p1, cg8, v0[3]);
      y1[0] = fmaf(p2, cg, v1[0]);  y1[1] = fmaf(p3, cg, v1[1]);
      y1[2] = fmaf(p2, cg8, v1[2]); y1[3] = fmaf(p3, cg8, v1[3]);
      // carry for the next block: the UNCORRECTED last token (btp-forward.cu:297-299)
      const int src = lane | 3;
      const float ng = __shfl_sync(0xffffffffu, v1[1], src);
      const float ng8 = __shfl_sync(0xffffffffu, v1[3], src);
      if constexpr (CKPT) {
        const int tile_in_seq = c.cs * (TL / 16) + i;
        const int tiles_per_seq = p.L >> 4;
        if (p.use_carry && tl.t == 3 && tile_in_seq < tiles_per_seq - 1) {
          float* dst = p.ckpt + (static_cast<long long>(c.bh) * tiles_per_seq + tile_in_seq) * 16;
          dst[tl.g] = v1[1];
          dst[tl.g + 8] = v1[3];
        }
      }
      if (p.use_carry) { cg = ng; cg8 = ng8; }
      if constexpr (OUT_F32) {
        float* yo = reinterpret_cast<float*>(p.out_f32) +
                    (static_cast<long long>(c.bh) * 16 + tl.g) * p.L + c.c0 + 16 * i + 2 * tl.t;
        const long long r8 = 8ll * p.L;
        *reinterpret_cast<float2*>(yo) = make_float2(y0[0], y0[1]);
        *reinterpret_cast<float2*>(yo + r8) = make_float2(y0[2], y0[3]);
        *reinterpret_cast<float2*>(yo + 8) = make_float2(y1[0], y1[1]);
        *reinterpret_cast<float2*>(yo + r8 + 8) = make_float2(y1[2], y1[3]);
      } else {
        __syncwarp();  // all lanes have consumed this block's x before it is overwritten
        const uint32_t o0 = tl.frag_addr(box_base, ib, 0);
        const uint32_t o1 = tl.frag_addr(box_base, ib, 1);
        st_shared_u32(o0, pack_bf16x2(y0[0], y0[1]));
        st_shared_u32(o0 + 1024, pack_bf16x2(y0[2], y0[3]));
        st_shared_u32(o1, pack_bf16x2(y1[0], y1[1]));
        st_shared_u32(o1 + 1024, pack_bf16x2(y1[2], y1[3]));
      }
    }
    if constexpr (!OUT_F32) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int nbox = (c.nt + 3) >> 2;
        for (int b = 0; b < nbox; ++b) tma_store_2d(&tm_y, c.c0 + 64 * b, c.bh * 16, ws.x(s) + b * 2048);
        bulk_commit_group();
      }
    } else {
      __syncwarp();  // T of this stage is free again
    }
  }

  if (failed) {
    if (lane == 0) report_timeout(warp, cb + pending_from);
    // give the loads still in flight a (bounded) chance to land before the buffers are released
    for (int j = pending_from; j < n && j < pending_from + AHEAD + 1; ++j) {
      mbar_wait_bounded(ws.bar(j % STAGES), (j / STAGES) & 1, kWaitLimitNs);
    }
  }
  if (!OUT_F32 && lane == 0) bulk_wait_group<0>();
}

// =====================================================================================
// Backward
// =====================================================================================
struct TileAcc {
  float v0[4], v1[4];  // local pass   v  (channels g / g+8 x tokens 2t,2t+1 | 8+2t,9+2t)
  float g0[4], g1[4];  // gw = dy . Lmat
};

struct PendingTile {
  int stage;
  int i;            // block inside its chunk
  float cg, cg8;    // carry INTO this block
  bool seq_end;     // last block of its sequence: no gradient arrives from the right
  bool chunk_end;   // last block of its chunk: outputs of the chunk are complete after it
  int bh, c0, nt;   // chunk coordinates, for the stores
};

template <int COEF, bool DY_F32, int NBOX, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
btp_backward_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                    const __grid_constant__ CUtensorMap tm_dx, const KernelParams p) {
  using LAYOUT = SmemLayout<NBOX, STAGES, WARPS, true, DY_F32>;
  constexpr int TL = LAYOUT::kTL;
  constexpr int kEsz = CoefTraits<COEF>::kBytes;
  static_assert(STAGES >= 3, "the backward ring needs three stages");

  extern __shared__ unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const WarpSmem<LAYOUT, STAGES> ws = carve_smem<LAYOUT, STAGES, WARPS>(smem_raw, warp);
  const TileLane tl(lane);

  const long long nwarps = static_cast<long long>(gridDim.x) * WARPS;
  const long long wid = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const int cb = static_cast<int>((wid * p.total_chunks) / nwarps);
  const int ce = static_cast<int>(((wid + 1) * p.total_chunks) / nwarps);
  const int n = ce - cb;
  if (n <= 0) return;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(ws.bar(s), 1);
    mbar_init_fence();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_dy);
    prefetch_tensormap(&tm_dx);
  }
  __syncwarp();

  auto issue = [&](int j) {
    const ChunkPos c = chunk_pos<TL>(cb + j, p.ncs, p.L);
    const int s = j % STAGES;
    const int nbox = (c.nt + 3) >> 2;
    const int nbox_dy = DY_F32 ? (c.nt + 1) >> 1 : nbox;
    const uint32_t cbytes = c.nt * 16 * kEsz;
    mbar_arrive_expect_tx(ws.bar(s), (nbox + nbox_dy) * 2048 + cbytes);
    for (int b = 0; b < nbox; ++b) tma_load_2d(ws.x(s) + b * 2048, &tm_x, c.c0 + 64 * b, c.bh * 16, ws.bar(s));
    for (int b = 0; b < nbox_dy; ++b)
      tma_load_2d(ws.dy(s) + b * 2048, &tm_dy, c.c0 + (DY_F32 ? 32 : 64) * b, c.bh * 16, ws.bar(s));
    bulk_load(ws.t_addr(s), reinterpret_cast<const char*>(p.coeff) + (static_cast<long long>(c.bh) * p.L + c.c0) * kEsz,
              cbytes, ws.bar(s));
  };

  // Chunk j's outputs leave one block into chunk j+1 (its last block needs the gradient that
  // arrives from the right).  Stage of chunk j is reloaded with chunk j+STAGES one chunk later
  // still, when that store has certainly drained: loads run STAGES-2 chunks ahead.
  int issued = 0;  // uniform across the warp; only lane 0 acts on it
  for (; issued < STAGES - 1 && issued < n; ++issued) {
    if (lane == 0) issue(issued);
  }

  // Front half of a block: tensor-core products.  Back half: everything that needs dCarry.
  auto front = [&](int s, int i, TileAcc& acc, float& dc_g, float& dc_g8) {
    const int box = i >> 2, ib = i & 3;
    const float* Tt = ws.t_ptr(s) + 16 * i;
    float2 Ta, Tb;
    const LmatFrag lf = build_lmat(Tt, tl, Ta, Tb);
    // dy . Lmat needs the transposed 8x8 blocks as B operand (k = r, n = c)
    const uint32_t g00 = movmatrix_trans(lf.b00);
    const uint32_t g10 = movmatrix_trans(lf.b10);
    const uint32_t g11 = movmatrix_trans(lf.b11);
    uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
    ldmatrix_x4(tl.ldm_addr(ws.x(s) + box * 2048, ib), a0, a1, a2, a3);
    if constexpr (DY_F32) {
      // [16][32] float boxes, 128-byte swizzle: block i sits in box i/2 at 64-byte offset (i&1)*64
      const uint32_t bb = ws.dy(s) + (i >> 1) * 2048 + tl.g * 128;
      const uint32_t c_lo = ((i & 1) * 4 + (tl.t >> 1)), c_hi = c_lo + 2;
      const uint32_t in = (tl.t & 1) * 8;
      float2 f;
      auto lds = [&](uint32_t addr) {
        float2 r;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(r.x), "=f"(r.y) : "r"(addr));
        return r;
      };
      f = lds(bb + ((c_lo ^ tl.g) << 4) + in);         e0 = pack_bf16x2(f.x, f.y);
      f = lds(bb + 1024 + ((c_lo ^ tl.g) << 4) + in);  e1 = pack_bf16x2(f.x, f.y);
      f = lds(bb + ((c_hi ^ tl.g) << 4) + in);         e2 = pack_bf16x2(f.x, f.y);
      f = lds(bb + 1024 + ((c_hi ^ tl.g) << 4) + in);  e3 = pack_bf16x2(f.x, f.y);
    } else {
      ldmatrix_x4(tl.ldm_addr(ws.dy(s) + box * 2048, ib), e0, e1, e2, e3);
    }
    mma_1688(acc.v0, a0, a1, lf.b00);
    mma_16816(acc.v1, a0, a1, a2, a3, lf.b10, lf.b11);
    mma_16816(acc.g0, e0, e1, e2, e3, g00, g10);
    mma_1688(acc.g1, e2, e3, g11);
    // gradient this block sends to its left neighbour: a_0 * gw[:,0]
    const float a_first = ex2(Tt[0]);
    const int src = lane & ~3;
    dc_g = a_first * __shfl_sync(0xffffffffu, acc.g0[0], src);
    dc_g8 = a_first * __shfl_sync(0xffffffffu, acc.g0[2], src);
  };

  auto back = [&](const PendingTile& pt, const TileAcc& acc, float dc_g, float dc_g8) {
    const int s = pt.stage, i = pt.i;
    const int box = i >> 2, ib = i & 3;
    const float* Tt = ws.t_ptr(s) + 16 * i;
    const float2 Ta = *reinterpret_cast<const float2*>(Tt + 2 * tl.t);
    const float2 Tb = *reinterpret_cast<const float2*>(Tt + 8 + 2 * tl.t);
    const float T15 = Tt[15];
    const float Tm1 = tl.t ? Tt[2 * tl.t - 1] : 0.0f;  // P[-1] = 1
    const float T7 = Tt[2 * tl.t + 7];
    const float l0 = ex2(T15 - Ta.x), l1 = ex2(T15 - Ta.y), l2 = ex2(T15 - Tb.x), l3 = ex2(T15 - Tb.y);
    float dx0[4], dx1[4];
    dx0[0] = fmaf(l0, dc_g, acc.g0[0]);  dx0[1] = fmaf(l1, dc_g, acc.g0[1]);
    dx0[2] = fmaf(l0, dc_g8, acc.g0[2]); dx0[3] = fmaf(l1, dc_g8, acc.g0[3]);
    dx1[0] = fmaf(l2, dc_g, acc.g1[0]);  dx1[1] = fmaf(l3, dc_g, acc.g1[1]);
    dx1[2] = fmaf(l2, dc_g8, acc.g1[2]); dx1[3] = fmaf(l3, dc_g8, acc.g1[3]);
    // v shifted right by one token
    const int src = (lane & ~3) | ((lane + 3) & 3);
    const float A_g = __shfl_sync(0xffffffffu, acc.v0[1], src);
    const float A_g8 = __shfl_sync(0xffffffffu, acc.v0[3], src);
    const float B_g = __shfl_sync(0xffffffffu, acc.v1[1], src);
    const float B_g8 = __shfl_sync(0xffffffffu, acc.v1[3], src);
    const float vp0_g = tl.t ? A_g : 0.0f, vp0_g8 = tl.t ? A_g8 : 0.0f;
    const float vp2_g = tl.t ? B_g : A_g, vp2_g8 = tl.t ? B_g8 : A_g8;
    const float pc0 = ex2(Tm1), pc1 = ex2(Ta.x), pc2 = ex2(T7), pc3 = ex2(Tb.x);
    const float cg = pt.cg, cg8 = pt.cg8;
    float m0 = fmaf(vp0_g, dx0[0], vp0_g8 * dx0[2]);
    float m1 = fmaf(acc.v0[0], dx0[1], acc.v0[2] * dx0[3]);
    float m2 = fmaf(vp2_g, dx1[0], vp2_g8 * dx1[2]);
    float m3 = fmaf(acc.v1[0], dx1[1], acc.v1[2] * dx1[3]);
    m0 = fmaf(pc0, fmaf(acc.g0[0], cg, acc.g0[2] * cg8), m0);
    m1 = fmaf(pc1, fmaf(acc.g0[1], cg, acc.g0[3] * cg8), m1);
    m2 = fmaf(pc2, fmaf(acc.g1[0], cg, acc.g1[2] * cg8), m2);
    m3 = fmaf(pc3, fmaf(acc.g1[1], cg, acc.g1[3] * cg8), m3);
    // sum over the 16 channels: channel pairs are in-thread, the 8 groups g are folded by a
    // transposing butterfly (each step halves the number of tokens a lane keeps)
    const bool b0 = (tl.g & 1) != 0, b1 = (tl.g & 2) != 0;
    const float keep0 = b0 ? m2 : m0, keep1 = b0 ? m3 : m1;
    const float send0 = b0 ? m0 : m2, send1 = b0 ? m1 : m3;
    const float r0 = keep0 + __shfl_xor_sync(0xffffffffu, send0, 4);
    const float r1 = keep1 + __shfl_xor_sync(0xffffffffu, send1, 4);
    const float keep = b1 ? r1 : r0, send = b1 ? r0 : r1;
    float r = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    r += __shfl_xor_sync(0xffffffffu, r, 16);
    if (lane < 16) {
      // token kept by this lane: [2t, 2t+1, 2t+8, 2t+9][2*b0 + b1]
      const int tok = 2 * tl.t + (b1 ? 1 : 0) + (b0 ? 8 : 0);
      float val = r;
      if constexpr (COEF == kCoefF32Log) {
        // gradient w.r.t. the log coefficient: dA * a,  a_tok = 2^(T_tok - T_{tok-1})
        const float Tprev = tok ? Tt[tok - 1] : 0.0f;
        val *= ex2(Tt[tok] - Tprev);
      }
      ws.da_ptr(s)[16 * i + tok] = val;
    }
    // dx replaces the consumed x block in shared memory
    const uint32_t box_base = ws.x(s) + box * 2048;
    const uint32_t o0 = tl.frag_addr(box_base, ib, 0);
    const uint32_t o1 = tl.frag_addr(box_base, ib, 1);
    st_shared_u32(o0, pack_bf16x2(dx0[0], dx0[1]));
    st_shared_u32(o0 + 1024, pack_bf16x2(dx0[2], dx0[3]));
    st_shared_u32(o1, pack_bf16x2(dx1[0], dx1[1]));
    st_shared_u32(o1 + 1024, pack_bf16x2(dx1[2], dx1[3]));
  };

  auto flush = [&](const PendingTile& pt) {  // chunk complete: send dx and dA on their way
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      const int nbox = (pt.nt + 3) >> 2;
      for (int b = 0; b < nbox; ++b) tma_store_2d(&tm_dx, pt.c0 + 64 * b, pt.bh * 16, ws.x(pt.stage) + b * 2048);
      bulk_store(p.dA + static_cast<long long>(pt.bh) * p.L + pt.c0, ws.da_addr(pt.stage), pt.nt * 64);
      bulk_commit_group();
      if (issued < n) {
        // the next load goes into the stage of the chunk flushed one chunk earlier
        bulk_wait_group_read<1>();
        issue(issued);
      }
    }
    if (issued < n) ++issued;
  };

  TileAcc cur, nxt;
  PendingTile pend;
  bool have = false;
  bool failed = false;
  int fail_chunk = 0;
  float vl_g = 0.0f, vl_g8 = 0.0f;  // uncorrected last token of the most recent block

  for (int j = 0; j < n && !failed; ++j) {
    const int s = j % STAGES;
    const ChunkPos c = chunk_pos<TL>(cb + j, p.ncs, p.L);
    if (!mbar_wait_bounded(ws.bar(s), (j / STAGES) & 1, kWaitLimitNs)) {
      failed = true;
      fail_chunk = j;
      break;
    }
    coeff_to_prefix<COEF, TL>(ws.t_ptr(s), lane);
    if (j == 0 && c.cs != 0 && p.use_carry) {
      halo_reduce<COEF, false, false>(p.x, p.coeff, p.L, c.bh, c.c0 - 16, lane, vl_g, vl_g8);
    }
    for (int i = 0; i < c.nt; ++i) {
      float dc_g, dc_g8;
      __syncwarp();
      front(s, i, nxt, dc_g, dc_g8);
      if (have) {
        const bool cut = pend.seq_end || !p.use_carry;
        back(pend, cur, cut ? 0.0f : dc_g, cut ? 0.0f : dc_g8);
        if (pend.chunk_end) flush(pend);
      }
      const bool seq_start = (c.cs == 0 && i == 0);
      pend.stage = s;
      pend.i = i;
      pend.cg = (seq_start || !p.use_carry) ? 0.0f : vl_g;
      pend.cg8 = (seq_start || !p.use_carry) ? 0.0f : vl_g8;
      pend.seq_end = (c.cs == p.ncs - 1) && (i == c.nt - 1);
      pend.chunk_end = (i == c.nt - 1);
      pend.bh = c.bh;
      pend.c0 = c.c0;
      pend.nt = c.nt;
      cur = nxt;
      have = true;
      const int src = lane | 3;
      vl_g = __shfl_sync(0xffffffffu, cur.v1[1], src);
      vl_g8 = __shfl_sync(0xffffffffu, cur.v1[3], src);
    }
  }

  if (!failed && have) {
    float dc_g = 0.0f, dc_g8 = 0.0f;
    if (!pend.seq_end && p.use_carry) {
      // the block to the right belongs to another warp: recompute what it sends
      halo_reduce<COEF, DY_F32, true>(p.dy, p.coeff, p.L, pend.bh, pend.c0 + 16 * pend.nt, lane, dc_g, dc_g8);
    }
    back(pend, cur, dc_g, dc_g8);
    flush(pend);
  }
  if (failed) {
    if (lane == 0) report_timeout(warp, cb + fail_chunk);
    for (int j = fail_chunk; j < issued; ++j) mbar_wait_bounded(ws.bar(j % STAGES), (j / STAGES) & 1, kWaitLimitNs);
  }
  if (lane == 0) bulk_wait_group<0>();
}

}  // namespace btp
