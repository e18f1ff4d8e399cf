// Backward of the gated BTP in token-major layout (see btp_gated.cuh for the forward and the data flow).
//
// Inputs  A_logits [B,L,H], B_logits, C, V, dOut [B,L,H*16]        (bf16, token-major)
// Outputs dA_logits [B,L,H], dB_logits, dC, dV [B,L,H*16]          (bf16, token-major)
//   sigma = bf16(sigmoid(B_logits))      x  = bf16(sigma * V)       a = bf16(sigmoid(A_logits))
//   y  = btp(a, x)   (recomputed)        dy = bf16(dOut * C)        (dx, dA) = btp_backward(a, x, dy)
//   dC = dOut * y    dV = dOut + dx * sigma    dB_logits = dx * V * sigma (1 - sigma)    dA_logits = dA * a (1 - a)
// Replaces autograd through spear/nn/phalanx/swr.py:216-219, 320-323, the transposing copies of
// spear/ops/btp/interface.py:186-187 and spear._btp.backward: about twenty passes over the activations.
//
// One CTA = 4 warps = 4 neighbouring heads; a work unit is a chunk of 32 tokens: four TMA boxes
// [32 tokens][64 channels] (B_logits, C, V, dOut).  dB, dC, dV overwrite their inputs in shared memory and
// leave with TMA stores.  As in the plain backward kernel, a block is finished one block later (it needs
// the gradient that its right neighbour sends), so a block's operands and accumulators wait in registers.
//
// Shared key/value heads (SHARED == true): B_logits and C are [B, L, kv_heads*16] and are read in place, each
// warp fetching its key/value head's 16 columns as a dense tile of its own (see btp_gated.cuh).  Each warp
// overwrites its tile with its head's dB_logits / dC; before they leave, the CTA sums the tiles of neighbouring
// heads that share a key/value head: runs of r = 4 heads when the group size is a multiple of 4, of r = 2 when it
// is 2, none otherwise.  The outputs are [B, L, H*16/r]: already the gradient of the key/value head when
// r equals the group size, else partial sums that the caller adds up (group/r of them per key/value head).
#pragma once

#include "btp_gated.cuh"

namespace btp {

struct GatedBwdParams {
  const __nv_bfloat16* a_logits;
  const __nv_bfloat16* b_logits;
  const __nv_bfloat16* c;
  const __nv_bfloat16* v;
  const __nv_bfloat16* dout;
  __nv_bfloat16* da_logits;
  long long ld_a, ld_b, ld_c, ld_v, ld_do, ld_da;  // row pitches in elements
  int L, H, hgs, ncs, total_units, use_carry, interleave;
  int group;  // heads per key/value head (see btp_gated.cuh); 1 when every head has its own
  unsigned long long wait_limit_ns;  // bounded waits give up after this long
};

constexpr int kGbTL = 32;            // tokens per chunk
constexpr int kGbBox = 32 * 128;     // bytes of one [32 tokens][64 channels] bf16 box
constexpr int kGbTables = 5;         // T, P, Pshift, L15, S = a (1 - a)

template <int STAGES>
struct GatedBwdSmem {
  static constexpr int kIo = 3 * STAGES * kGbBox;            // B, C, V rings (outputs in place)
  static constexpr int kDo = (STAGES - 1) * kGbBox;          // dOut ring
  static constexpr int kTab = 4 * 2 * kGbTables * kGbTL * 4;  // per warp, two sets
  static constexpr int kDa = 2 * kGbTL * 4 * 2;               // dA_logits staging [2][32 tokens][4 heads] bf16
  static constexpr int kBytes = kIo + kDo + kTab + kDa + STAGES * 8;
};

// Gradient that the 16-token block starting at `tok0` sends to its left neighbour, recomputed from global
// memory: dCarry[ch] = P[0] * sum_r dy[ch,r] * bf16(2^(T_r - T_0)),  dy = bf16(dOut * C).
__device__ __forceinline__ void gated_halo_right(const GatedBwdParams& p, long long b, int h, int tok0, int lane,
                                                 float& out_g, float& out_g8) {
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = b * p.L + tok0;
  float T = logit_to_log2a(__bfloat162float(p.a_logits[(row0 + (lane & 15)) * p.ld_a + h]));
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, T, d, 16);
    if ((lane & 15) >= d) T += up;
  }
  const float T0 = __shfl_sync(0xffffffffu, T, 0);
  float sg = 0.0f, sg8 = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tok = 2 * t + (j & 1) + ((j >> 1) << 3);
    const float w = lmat_weight<true>(ex2(__shfl_sync(0xffffffffu, T, tok) - T0));
    const long long rd = (row0 + tok) * p.ld_do + h * 16;
    const long long rc = (row0 + tok) * p.ld_c + (h / p.group) * 16;
    const float dy_g = round_bf16(__bfloat162float(p.dout[rd + g]) * __bfloat162float(p.c[rc + g]));
    const float dy_g8 = round_bf16(__bfloat162float(p.dout[rd + g + 8]) * __bfloat162float(p.c[rc + g + 8]));
    sg = fmaf(dy_g, w, sg);
    sg8 = fmaf(dy_g8, w, sg8);
  }
  sg += __shfl_xor_sync(0xffffffffu, sg, 1);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 1);
  sg += __shfl_xor_sync(0xffffffffu, sg, 2);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 2);
  const float a0 = ex2(T0);
  out_g = sg * a0;
  out_g8 = sg8 * a0;
}

// What a block keeps in registers until its right neighbour has been multiplied.
struct GatedPending {
  float v0[4], v1[4];  // local pass v
  float g0[4], g1[4];  // gw = dy . Lmat
  uint32_t sp[4];      // sigma, packed bf16 (operand arrangement: ch g | g+8, tokens 2t.. | 8+2t..)
  uint32_t vf[4];      // V
  uint32_t df[4];      // dOut
};

// Sums the [TL][16] bf16 tiles of each run of R neighbouring heads into the run's first tile, in float32.  A tile is
// TL*32 bytes = 128 units of 8 bytes = one unit per thread; a thread reads its unit from the R tiles of a run and
// writes it back to the first of them, so no thread touches another thread's unit.
template <int R>
__device__ __forceinline__ void sum_head_tiles(unsigned char* slot, int tid) {
  static_assert(kGbTL * 32 == 128 * 8, "one 8-byte unit of a tile per thread");
#pragma unroll
  for (int run = 0; run < 4 / R; ++run) {
    uint2* first = reinterpret_cast<uint2*>(slot + run * R * (kGbTL * 32)) + tid;
    const uint2 v = *first;
    float s0 = bf16_lo(v.x), s1 = bf16_hi(v.x), s2 = bf16_lo(v.y), s3 = bf16_hi(v.y);
#pragma unroll
    for (int q = 1; q < R; ++q) {
      const uint2 o = *(reinterpret_cast<const uint2*>(slot + (run * R + q) * (kGbTL * 32)) + tid);
      s0 += bf16_lo(o.x); s1 += bf16_hi(o.x); s2 += bf16_lo(o.y); s3 += bf16_hi(o.y);
    }
    *first = make_uint2(pack_bf16x2(s0, s1), pack_bf16x2(s2, s3));
  }
}

// REDUCE: shared heads only - dB_logits / dC are summed over runs of this many neighbouring heads (1, 2 or 4).
template <int STAGES, bool SHARED, int REDUCE = 1>
__global__ void __launch_bounds__(128, 4)
btp_gated_backward_kernel(const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                          const __grid_constant__ CUtensorMap tm_db, const __grid_constant__ CUtensorMap tm_dc,
                          const __grid_constant__ CUtensorMap tm_dv, const GatedBwdParams p) {
  static_assert(STAGES >= 3, "compute, draining stores and load in flight need three stages");
  constexpr int TL = kGbTL;
  using SM = GatedBwdSmem<STAGES>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const TileLane tl(lane);

  const WarpWork work(blockIdx.x, gridDim.x, p.total_units, p.ncs, p.interleave != 0);
  const int n = work.n;
  if (n <= 0) return;
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0) {
    if (tid == 0) report_error(2u, warp, 0);
    return;
  }
  auto io_addr = [&](int which, int s) { return base + (which * STAGES + s) * kGbBox; };  // 0 B, 1 C, 2 V
  auto do_addr = [&](int d) { return base + SM::kIo + d * kGbBox; };
  float* tab_base = reinterpret_cast<float*>(smem_raw + SM::kIo + SM::kDo) + warp * 2 * kGbTables * TL;
  __nv_bfloat16* da_stage = reinterpret_cast<__nv_bfloat16*>(smem_raw + SM::kIo + SM::kDo + SM::kTab);
  const uint32_t bars = base + SM::kIo + SM::kDo + SM::kTab + SM::kDa;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
    mbar_init_fence();
    fence_proxy_async_smem();
  }
  __syncthreads();

  const int L = p.L, ncs = p.ncs, hgs = p.hgs;
  const float carry_scale = p.use_carry ? 1.0f : 0.0f;
  GatedCursor prod(work.bh, work.cs, work.step, hgs), cons(work.bh, work.cs, work.step, hgs);
  int s_prod = 0, d_prod = 0, issued = 0;
  auto issue = [&]() {
    if constexpr (SHARED) {
      // threads 0-3: B_logits tiles of heads 0-3, 4-7: their C tiles, 8: V box, 9: dOut box; one copy instruction
      if (tid < 10) {
        const uint32_t bar = bars + s_prod * 8;
        if (tid == 0) mbar_arrive_expect_tx(bar, 4 * kGbBox);
        const int w = tid & 3;
        const int kv_col = ((prod.hg * 4 + w) / p.group) * 16;
        const uint64_t map = reinterpret_cast<uint64_t>(tid < 4 ? &tm_b : (tid < 8 ? &tm_c : (tid == 8 ? &tm_v : &tm_do)));
        const uint32_t to = tid < 8 ? io_addr(tid >> 2, s_prod) + w * (TL * 32) : (tid == 8 ? io_addr(2, s_prod) : do_addr(d_prod));
        tma_load_3d(to, map, tid < 8 ? kv_col : prod.hg * 64, prod.cs * TL, prod.b, bar);
      }
    } else if (tid == 0) {
      const uint32_t bar = bars + s_prod * 8;
      const int col = prod.hg * 64, row = prod.cs * TL;
      mbar_arrive_expect_tx(bar, 4 * kGbBox);
      tma_load_3d(io_addr(0, s_prod), &tm_b, col, row, prod.b, bar);
      tma_load_3d(io_addr(1, s_prod), &tm_c, col, row, prod.b, bar);
      tma_load_3d(io_addr(2, s_prod), &tm_v, col, row, prod.b, bar);
      tma_load_3d(do_addr(d_prod), &tm_do, col, row, prod.b, bar);
    }
    prod.next(ncs, hgs);
    s_prod = (s_prod + 1 == STAGES) ? 0 : s_prod + 1;
    d_prod = (d_prod + 1 == STAGES - 1) ? 0 : d_prod + 1;
    ++issued;
  };
  auto load_logit = [&](const GatedCursor& c) {  // the one logit this lane owns in a chunk
    const int tok = c.cs * TL + lane;
    const long long row = static_cast<long long>(c.b) * L + tok;
    return (tok < L) ? __bfloat162float(p.a_logits[row * p.ld_a + c.hg * 4 + warp]) : 0.0f;
  };
  while (issued < STAGES - 1 && issued < n) issue();
  // the logits run two chunks ahead of the consumer: a 32-token chunk is too short to hide a global load
  GatedCursor peek = cons;
  float z_next = load_logit(peek), z_after = 0.0f;
  peek.next(ncs, hgs);
  if (n > 1) {
    z_after = load_logit(peek);
    peek.next(ncs, hgs);
  }

  const uint32_t frag_off = ((lane & 7) + 8 * (lane >> 4)) * 128 + (((2 * warp + ((lane >> 3) & 1)) ^ (lane & 7)) << 4);
  // the same block inside this warp's dense [TL][16 channels] tile (shared key/value heads)
  const uint32_t kv_off = SHARED ? warp * (TL * 32) + ((lane & 7) + 8 * (lane >> 4)) * 32 + ((((lane >> 3) ^ (lane >> 2)) & 1) << 4) : frag_off;
  constexpr uint32_t kKvBlock = SHARED ? 512 : 2048;  // bytes from one 16-token block to the next in the B / C tiles

  // ---- per chunk: tables T, P, Pshift, L15, S (one token per lane, 16 lanes per block)
  auto make_tables = [&](float z, float* tab) {
    const float a = round_bf16(rcp_approx(1.0f + ex2(-z * kLog2E)));
    float T = (a > kTinyCoeff) ? lg2(a) : kZeroLog2;
    const int q = lane & 15;
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, T, d, 16);
      if (q >= d) T += up;
    }
    const float P = ex2(T);
    float prev = __shfl_up_sync(0xffffffffu, P, 1, 16);
    if (q == 0) prev = 1.0f;
    const float T15 = __shfl_sync(0xffffffffu, T, lane | 15);
    __syncwarp();
    tab[lane] = T;
    tab[TL + lane] = P * carry_scale;
    tab[2 * TL + lane] = prev * carry_scale;
    tab[3 * TL + lane] = ex2(T15 - T);
    tab[4 * TL + lane] = a * (1.0f - a);
    __syncwarp();
  };

  // ---- front half of a block: operands, the eight tensor-core products, dC
  auto front = [&](const float* tab, uint32_t sb, uint32_t sc, uint32_t sv, uint32_t sd, int i, float cg, float cg8,
                   GatedPending& pd, float& dc_g, float& dc_g8) {
    uint32_t bf[4], cf[4];
    ldmatrix_x4_trans(sb + kKvBlock * i, bf[0], bf[1], bf[2], bf[3]);
    ldmatrix_x4_trans(sv + 2048 * i, pd.vf[0], pd.vf[1], pd.vf[2], pd.vf[3]);
    ldmatrix_x4_trans(sc + kKvBlock * i, cf[0], cf[1], cf[2], cf[3]);
    ldmatrix_x4_trans(sd + 2048 * i, pd.df[0], pd.df[1], pd.df[2], pd.df[3]);
    uint32_t x[4], dy[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      pd.sp[r] = sigmoid_pair(bf[r]);
      x[r] = mul_bf16x2(pd.sp[r], pd.vf[r]);
      dy[r] = mul_bf16x2(pd.df[r], cf[r]);
    }
    const float* tg = tab + tl.g;
    const float* tt = tab + 2 * tl.t;
    LmatFrag lf, lo;
    build_lmat_split(tg, tt, 16 * i, tl, lf, lo);
    // the two 8-token products take their hi and lo terms in one k = 16 instruction each (left operand given twice)
    mma_16816(pd.v0, x[0], x[1], x[0], x[1], lf.b00, lo.b00);
    mma_16816(pd.v1, x[0], x[1], x[2], x[3], lf.b10, lf.b11);
    mma_16816_acc(pd.v1, x[0], x[1], x[2], x[3], lo.b10, lo.b11);
    mma_16816(pd.g0, dy[0], dy[1], dy[2], dy[3], movmatrix_trans(lf.b00), movmatrix_trans(lf.b10));
    mma_16816_acc(pd.g0, dy[0], dy[1], dy[2], dy[3], movmatrix_trans(lo.b00), movmatrix_trans(lo.b10));
    mma_16816(pd.g1, dy[2], dy[3], dy[2], dy[3], movmatrix_trans(lf.b11), movmatrix_trans(lo.b11));
    // y = v + P * carry;  dC = dOut * y
    const float2 Pa = *reinterpret_cast<const float2*>(tt + TL + 16 * i);
    const float2 Pb = *reinterpret_cast<const float2*>(tt + TL + 16 * i + 8);
    const uint32_t q0 = pack_bf16x2(bf16_lo(pd.df[0]) * fmaf(Pa.x, cg, pd.v0[0]), bf16_hi(pd.df[0]) * fmaf(Pa.y, cg, pd.v0[1]));
    const uint32_t q1 = pack_bf16x2(bf16_lo(pd.df[1]) * fmaf(Pa.x, cg8, pd.v0[2]), bf16_hi(pd.df[1]) * fmaf(Pa.y, cg8, pd.v0[3]));
    const uint32_t q2 = pack_bf16x2(bf16_lo(pd.df[2]) * fmaf(Pb.x, cg, pd.v1[0]), bf16_hi(pd.df[2]) * fmaf(Pb.y, cg, pd.v1[1]));
    const uint32_t q3 = pack_bf16x2(bf16_lo(pd.df[3]) * fmaf(Pb.x, cg8, pd.v1[2]), bf16_hi(pd.df[3]) * fmaf(Pb.y, cg8, pd.v1[3]));
    __syncwarp();  // every lane holds its C fragment before the block is overwritten
    stmatrix_x4_trans(sc + kKvBlock * i, q0, q1, q2, q3);
    // gradient this block sends to its left neighbour: P[0] * gw[:,0]
    const float p_first = tab[TL + 16 * i];
    dc_g = p_first * __shfl_sync(0xffffffffu, pd.g0[0], lane & ~3);
    dc_g8 = p_first * __shfl_sync(0xffffffffu, pd.g0[2], lane & ~3);
  };

  // ---- back half of a block: everything that needs the gradient arriving from the right.
  // tt_i = &T[16 i + 2t] of the block's table set, da_i = dA_logits staging of its chunk at token 16 i,
  // sb_i / sv_i = this warp's block inside the B and V boxes of its stage.
  auto back = [&](const GatedPending& pd, const float* tt_i, __nv_bfloat16* da_i, uint32_t sb_i, uint32_t sv_i,
                  float cg, float cg8, float dc_g, float dc_g8) {
    const float2 Sa = *reinterpret_cast<const float2*>(tt_i + 2 * TL);      // P[2t-1], P[2t]
    const float2 Sb = *reinterpret_cast<const float2*>(tt_i + 2 * TL + 8);  // P[2t+7], P[2t+8]
    const float2 La = *reinterpret_cast<const float2*>(tt_i + 3 * TL);      // Lmat[15, 2t], Lmat[15, 2t+1]
    const float2 Lb = *reinterpret_cast<const float2*>(tt_i + 3 * TL + 8);
    float dx[8];  // operand arrangement: [0,1] (g; 2t,2t+1) [2,3] (g+8; 2t,2t+1) [4,5] (g; 8+2t..) [6,7] (g+8; 8+2t..)
    dx[0] = fmaf(La.x, dc_g, pd.g0[0]);  dx[1] = fmaf(La.y, dc_g, pd.g0[1]);
    dx[2] = fmaf(La.x, dc_g8, pd.g0[2]); dx[3] = fmaf(La.y, dc_g8, pd.g0[3]);
    dx[4] = fmaf(Lb.x, dc_g, pd.g1[0]);  dx[5] = fmaf(Lb.y, dc_g, pd.g1[1]);
    dx[6] = fmaf(Lb.x, dc_g8, pd.g1[2]); dx[7] = fmaf(Lb.y, dc_g8, pd.g1[3]);
    // dA: v shifted right by one token
    const int src = (lane & ~3) | ((lane + 3) & 3);
    const float A_g = __shfl_sync(0xffffffffu, pd.v0[1], src);
    const float A_g8 = __shfl_sync(0xffffffffu, pd.v0[3], src);
    const float B_g = __shfl_sync(0xffffffffu, pd.v1[1], src);
    const float B_g8 = __shfl_sync(0xffffffffu, pd.v1[3], src);
    const float vp0_g = tl.t ? A_g : 0.0f, vp0_g8 = tl.t ? A_g8 : 0.0f;
    const float vp2_g = tl.t ? B_g : A_g, vp2_g8 = tl.t ? B_g8 : A_g8;
    float m0 = fmaf(vp0_g, dx[0], vp0_g8 * dx[2]);
    float m1 = fmaf(pd.v0[0], dx[1], pd.v0[2] * dx[3]);
    float m2 = fmaf(vp2_g, dx[4], vp2_g8 * dx[6]);
    float m3 = fmaf(pd.v1[0], dx[5], pd.v1[2] * dx[7]);
    m0 = fmaf(Sa.x, fmaf(pd.g0[0], cg, pd.g0[2] * cg8), m0);
    m1 = fmaf(Sa.y, fmaf(pd.g0[1], cg, pd.g0[3] * cg8), m1);
    m2 = fmaf(Sb.x, fmaf(pd.g1[0], cg, pd.g1[2] * cg8), m2);
    m3 = fmaf(Sb.y, fmaf(pd.g1[1], cg, pd.g1[3] * cg8), m3);
    const bool b0 = (tl.g & 1) != 0, b1 = (tl.g & 2) != 0;
    const float keep0 = b0 ? m2 : m0, keep1 = b0 ? m3 : m1;
    const float send0 = b0 ? m0 : m2, send1 = b0 ? m1 : m3;
    const float r0 = keep0 + __shfl_xor_sync(0xffffffffu, send0, 4);
    const float r1 = keep1 + __shfl_xor_sync(0xffffffffu, send1, 4);
    const float keep = b1 ? r1 : r0, send = b1 ? r0 : r1;
    float r = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    r += __shfl_xor_sync(0xffffffffu, r, 16);
    if (lane < 16) {
      const int tok = 2 * tl.t + (b1 ? 1 : 0) + (b0 ? 8 : 0);
      const float scale = (tt_i - 2 * tl.t)[4 * TL + tok];  // a (1 - a)
      da_i[tok * 4 + warp] = __float2bfloat16(r * scale);
    }
    // dV = dOut + dx * sigma,  dB_logits = dx * V * sigma (1 - sigma)
    uint32_t ov[4], ob[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float s_lo = bf16_lo(pd.sp[q]), s_hi = bf16_hi(pd.sp[q]);
      const float x_lo = dx[2 * q], x_hi = dx[2 * q + 1];
      ov[q] = pack_bf16x2(fmaf(x_lo, s_lo, bf16_lo(pd.df[q])), fmaf(x_hi, s_hi, bf16_hi(pd.df[q])));
      ob[q] = pack_bf16x2(x_lo * bf16_lo(pd.vf[q]) * fmaf(-s_lo, s_lo, s_lo), x_hi * bf16_hi(pd.vf[q]) * fmaf(-s_hi, s_hi, s_hi));
    }
    stmatrix_x4_trans(sv_i, ov[0], ov[1], ov[2], ov[3]);
    stmatrix_x4_trans(sb_i, ob[0], ob[1], ob[2], ob[3]);
  };

  GatedPending pa, pb;  // slot B holds the pending block at chunk boundaries
  bool have = false, failed = false, p_seq_end = false;
  const float* p_tt = nullptr;
  __nv_bfloat16* p_da = nullptr;
  uint32_t p_sb = 0, p_sv = 0;
  float p_cg = 0.0f, p_cg8 = 0.0f, vl_g = 0.0f, vl_g8 = 0.0f;
  int p_stage = 0, p_set = 0, p_b = 0, p_hg = 0, p_c0 = 0, p_nt = 0;

  // the pending block's chunk is complete: all four heads' dB, dC, dV boxes and the dA_logits rows leave
  auto flush = [&]() {
    fence_proxy_async_smem();
    __syncthreads();
    if constexpr (SHARED) {
      constexpr int r = REDUCE;
      if constexpr (REDUCE > 1) {
        sum_head_tiles<REDUCE>(smem_raw + (0 * STAGES + p_stage) * kGbBox, tid);  // dB_logits
        sum_head_tiles<REDUCE>(smem_raw + (1 * STAGES + p_stage) * kGbBox, tid);  // dC
        fence_proxy_async_smem();
        __syncthreads();
      }
      // threads 0-3: the dB tiles, 4-7: the dC tiles (16 columns each; only the first tile of every run of r heads
      // leaves), 8: the dV box; every storing thread keeps its own async group
      if (tid < 9) {
        const int w = tid & 3;
        const uint64_t map = reinterpret_cast<uint64_t>(tid < 4 ? &tm_db : (tid < 8 ? &tm_dc : &tm_dv));
        const uint32_t from = tid < 8 ? io_addr(tid >> 2, p_stage) + w * (TL * 32) : io_addr(2, p_stage);
        if (tid == 8 || w % r == 0)
          tma_store_3d(map, tid < 8 ? ((p_hg * 4 + w) / r) * 16 : p_hg * 64, p_c0, p_b, from);
        bulk_commit_group();
        if (issued < n) bulk_wait_group_read<1>();
      }
    } else if (tid == 0) {
      tma_store_3d(&tm_db, p_hg * 64, p_c0, p_b, io_addr(0, p_stage));
      tma_store_3d(&tm_dc, p_hg * 64, p_c0, p_b, io_addr(1, p_stage));
      tma_store_3d(&tm_dv, p_hg * 64, p_c0, p_b, io_addr(2, p_stage));
      bulk_commit_group();
      if (issued < n) bulk_wait_group_read<1>();  // the stores flushed one chunk earlier have drained
    }
    if (tid < TL && p_c0 + tid < L) {
      const uint2 row = reinterpret_cast<const uint2*>(da_stage + p_set * TL * 4)[tid];
      *reinterpret_cast<uint2*>(p.da_logits + (static_cast<long long>(p_b) * L + p_c0 + tid) * p.ld_da + p_hg * 4) = row;
    }
    if (issued < n) issue();
  };

  int j = 0, s = 0, d = 0, tset = 0;
  uint32_t phase = 0;
  for (; j < n; ++j) {
    const float z = z_next;
    z_next = z_after;
    if (j + 2 < n) {
      z_after = load_logit(peek);
      peek.next(ncs, hgs);
    }
    const bool ok = mbar_wait_bounded(bars + s * 8, phase, p.wait_limit_ns);
    if (__syncthreads_or(!ok)) {
      failed = true;
      break;
    }
    const int c0 = cons.cs * TL;
    const int nt = ((L - c0) >> 4) < 2 ? ((L - c0) >> 4) : 2;
    float* tab = tab_base + tset * kGbTables * TL;
    make_tables(z, tab);
    if (j == 0 && cons.cs != 0 && p.use_carry) {
      GatedParams hp{};
      hp.a_logits = p.a_logits; hp.b_logits = p.b_logits; hp.v = p.v;
      hp.ld_a = p.ld_a; hp.ld_b = p.ld_b; hp.ld_v = p.ld_v; hp.L = L; hp.group = p.group;
      gated_halo_left(hp, cons.b, cons.hg * 4 + warp, c0 - 16, lane, vl_g, vl_g8);
    }
    const float* tt = tab + 2 * tl.t;
    __nv_bfloat16* da = da_stage + tset * TL * 4;
    const uint32_t sb = io_addr(0, s) + kv_off, sc = io_addr(1, s) + kv_off, sv = io_addr(2, s) + frag_off;
    const uint32_t sd = do_addr(d) + frag_off;
    const bool seq_first = (cons.cs == 0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (i < nt) {
        GatedPending& cur = (i & 1) ? pb : pa;
        const GatedPending& prev = (i & 1) ? pa : pb;
        const float ncg = (i == 0 && seq_first) ? 0.0f : vl_g;  // carry into block i
        const float ncg8 = (i == 0 && seq_first) ? 0.0f : vl_g8;
        float dc_g, dc_g8;
        front(tab, sb, sc, sv, sd, i, ncg, ncg8, cur, dc_g, dc_g8);
        if (i == 0) {
          if (have) {
            back(prev, p_tt, p_da, p_sb, p_sv, p_cg, p_cg8, p_seq_end ? 0.0f : dc_g, p_seq_end ? 0.0f : dc_g8);
            flush();
          }
        } else {
          back(prev, tt, da, sb, sv, p_cg, p_cg8, dc_g, dc_g8);
        }
        p_cg = ncg;
        p_cg8 = ncg8;
        vl_g = __shfl_sync(0xffffffffu, cur.v1[1], lane | 3);
        vl_g8 = __shfl_sync(0xffffffffu, cur.v1[3], lane | 3);
      }
    }
    if (nt == 1) pb = pa;
    have = true;
    p_seq_end = (cons.cs == ncs - 1);
    p_tt = tt + 16 * (nt - 1);
    p_da = da + 16 * (nt - 1) * 4;
    p_sb = sb + kKvBlock * (nt - 1);
    p_sv = sv + 2048 * (nt - 1);
    p_stage = s;
    p_set = tset;
    p_b = cons.b;
    p_hg = cons.hg;
    p_c0 = c0;
    p_nt = nt;
    cons.next(ncs, hgs);
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
      gated_halo_right(p, p_b, p_hg * 4 + warp, p_c0 + 16 * p_nt, lane, dc_g, dc_g8);
    }
    back(pb, p_tt, p_da, p_sb, p_sv, p_cg, p_cg8, dc_g, dc_g8);
    flush();
  }
  if (failed) {
    if (tid == 0) report_error(1u, warp, j);
    for (int k = j; k < issued; ++k) {
      mbar_wait_bounded(bars + s * 8, phase, p.wait_limit_ns);
      if (++s == STAGES) {
        s = 0;
        phase ^= 1u;
      }
    }
  }
  if (tid < (SHARED ? 9 : 1)) bulk_wait_group<0>();
}

}  // namespace btp
