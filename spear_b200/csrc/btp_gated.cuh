// Gated BTP in token-major layout: the Phalanx layer's glue around the op, fused into the kernel.
//
// The layer computes (spear/nn/phalanx/swr.py:196-221, 311-327), from the outputs of its projections,
//   a = sigmoid(A_logits)              [B, L, H]        decay
//   X = sigmoid(B_logits) * V          [B, L, H*16]     driving term
//   y = btp(a, X)                                        (after two transposing copies, interface.py:186-187)
//   out = y * C + V                    [B, L, H*16]     fed to proj_out
// with every tensor TOKEN-major, exactly as the GEMMs leave them.  This kernel reads A_logits, B_logits,
// C, V in that layout and writes `out` in that layout: the sigmoid, the products, the two layout changes
// and the epilogue never touch HBM.
//
// Mapping: one CTA = 4 warps = 4 neighbouring heads (64 channels = one 128-byte swizzle span); a work unit
// is a chunk of 64 tokens of those 4 heads: three TMA boxes [64 tokens][64 channels] (B_logits, C, V).
// Warp w owns head 4*hg + w: it pulls its [16 channels x 16 tokens] operand out of the token-major box with
// ldmatrix.trans, gates it in registers, runs the same tensor-core block product as the plain kernel, forms
// y*C+V in the accumulator layout and puts the result back over V with stmatrix.trans; one thread then
// stores the box.  The CTA walks along sequences, so the carry stays in registers; a CTA whose range starts
// inside a sequence recomputes the carry of the block to its left from global memory.
//
// Shared key/value heads (SHARED == true; KVRepeat, swr.py:96-103: head h reads key/value head h / group).
// B_logits and C are then [B, L, kv_heads*16] and are read IN PLACE: each warp fetches the 16 columns of its
// key/value head as its own dense [tokens][16 channels] tile (32-byte rows, 32-byte swizzle), so the heads of a group
// fetch the same global columns - once from HBM, the repeats from L2 - and nothing is repeated in memory.
#pragma once

#include "btp_kernels.cuh"

namespace btp {

struct GatedParams {
  const __nv_bfloat16* a_logits;  // [B*L, ld_a]  logit of head h in column h
  const __nv_bfloat16* b_logits;  // [B*L, ld_b]  (halo reads)
  const __nv_bfloat16* v;         // [B*L, ld_v]  (halo reads)
  long long ld_a, ld_b, ld_v;     // row pitches in elements
  int L;                          // tokens per sequence
  int H;                          // heads
  int hgs;                        // head groups (H / 4)
  int ncs;                        // chunks per sequence
  int total_units;                // B * hgs * ncs
  int use_carry;                  // k == 2
  int interleave;                 // deal whole sequences round-robin to the CTAs
  int group;                      // heads per key/value head: head h reads columns (h / group) * 16 of B_logits and C
  unsigned long long wait_limit_ns;  // bounded waits give up after this long (btp_sm100_set_wait_limit)
};

// TL = tokens per chunk (32 or 64): one box is [TL tokens][64 channels] bf16.
template <int TL, int STAGES>
struct GatedSmem {
  static constexpr int kBox = TL * 128;
  static constexpr int kStage = 3 * kBox;           // B_logits, C, V
  static constexpr int kTables = 4 * 2 * TL * 4;    // per warp: T, P
  static constexpr int kBytes = STAGES * kStage + kTables + STAGES * 8;
};

// log2 of the decay that the layer derives from one logit: a = bf16(sigmoid(z)), as the layer rounds it.
__device__ __forceinline__ float logit_to_log2a(float z) {
  const float a = round_bf16(rcp_approx(1.0f + ex2(-z * kLog2E)));
  return (a > kTinyCoeff) ? lg2(a) : kZeroLog2;
}

// The layer's driving term for a pair of packed bf16 values, rounded where the layer rounds
// (swr.py:217-219): sigma = bf16(sigmoid(b)), x = bf16(sigma * v).
__device__ __forceinline__ uint32_t sigmoid_pair(uint32_t b) {
  return pack_bf16x2(sigmoid_fast(bf16_lo(b)), sigmoid_fast(bf16_hi(b)));
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t gate_pair(uint32_t b, uint32_t v) { return mul_bf16x2(sigmoid_pair(b), v); }
__device__ __forceinline__ float gate_scalar(float b, float v) { return round_bf16(round_bf16(sigmoid_fast(b)) * v); }

// carry of the 16-token block that starts at `tok0` of batch entry b, head h, recomputed from global memory
__device__ __forceinline__ void gated_halo_left(const GatedParams& p, long long b, int h, int tok0, int lane,
                                                float& out_g, float& out_g8) {
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = b * p.L + tok0;
  float T = logit_to_log2a(__bfloat162float(p.a_logits[(row0 + (lane & 15)) * p.ld_a + h]));
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, T, d, 16);
    if ((lane & 15) >= d) T += up;
  }
  const float T15 = __shfl_sync(0xffffffffu, T, 15);
  float sg = 0.0f, sg8 = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tok = 2 * t + (j & 1) + ((j >> 1) << 3);
    const float w = lmat_weight<true>(ex2(T15 - __shfl_sync(0xffffffffu, T, tok)));
    const long long rb = (row0 + tok) * p.ld_b + (h / p.group) * 16;
    const long long rv = (row0 + tok) * p.ld_v + h * 16;
    const float x_g = gate_scalar(__bfloat162float(p.b_logits[rb + g]), __bfloat162float(p.v[rv + g]));
    const float x_g8 = gate_scalar(__bfloat162float(p.b_logits[rb + g + 8]), __bfloat162float(p.v[rv + g + 8]));
    sg = fmaf(x_g, w, sg);
    sg8 = fmaf(x_g8, w, sg8);
  }
  sg += __shfl_xor_sync(0xffffffffu, sg, 1);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 1);
  sg += __shfl_xor_sync(0xffffffffu, sg, 2);
  sg8 += __shfl_xor_sync(0xffffffffu, sg8, 2);
  out_g = sg;
  out_g8 = sg8;
}

// Position of a CTA's work unit: (batch entry, head group, chunk).
struct GatedCursor {
  int b, hg, cs;
  int step_b, step_hg;  // advance, in (b, hg) space, from one sequence of this CTA to its next
  __device__ __forceinline__ GatedCursor(int seq, int cs_, int step, int hgs)
      : b(seq / hgs), hg(seq - (seq / hgs) * hgs), cs(cs_), step_b(step / hgs), step_hg(step - (step / hgs) * hgs) {}
  __device__ __forceinline__ void next(int ncs, int hgs) {
    if (++cs == ncs) {
      cs = 0;
      b += step_b;
      hg += step_hg;
      if (hg >= hgs) {
        hg -= hgs;
        ++b;
      }
    }
  }
};

template <int TL, int STAGES, bool SHARED>
__global__ void __launch_bounds__(128)
btp_gated_forward_kernel(const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_out,
                         const GatedParams p) {
  static_assert(STAGES >= 3, "compute, draining store and load in flight need three stages");
  constexpr int TPL = TL / 32;  // tokens (logits) per lane and chunk
  constexpr int NT = TL / 16;   // blocks per chunk
  using SM = GatedSmem<TL, STAGES>;
  constexpr int kGatedBox = SM::kBox;
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
  const uint32_t bars = base + STAGES * SM::kStage + SM::kTables;
  float* tab = reinterpret_cast<float*>(smem_raw + STAGES * SM::kStage) + warp * 2 * TL;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
    mbar_init_fence();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_b);
    prefetch_tensormap(&tm_c);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_out);
  }
  __syncthreads();

  const int L = p.L, ncs = p.ncs, hgs = p.hgs;
  const float carry_scale = p.use_carry ? 1.0f : 0.0f;
  GatedCursor prod(work.bh, work.cs, work.step, hgs), cons(work.bh, work.cs, work.step, hgs);
  int s_prod = 0;
  auto issue = [&]() {
    const uint32_t dst = base + s_prod * SM::kStage;
    const uint32_t bar = bars + s_prod * 8;
    if constexpr (SHARED) {
      // thread 0: the V box (the thread that also stores `out` from that buffer), threads 1-4: the B_logits tiles
      // of heads 0-3, threads 5-8: their C tiles; one copy instruction for all nine.  The byte count is the same
      // as for three full boxes.
      if (tid < 9) {
        if (tid == 0) mbar_arrive_expect_tx(bar, 3 * kGatedBox);
        const int t = tid - 1, w = t & 3;
        const int kv_col = ((prod.hg * 4 + w) / p.group) * 16;
        const uint64_t map = reinterpret_cast<uint64_t>(tid == 0 ? &tm_v : (t < 4 ? &tm_b : &tm_c));
        const uint32_t to = tid == 0 ? dst + 2 * kGatedBox : dst + (t >> 2) * kGatedBox + w * (TL * 32);
        tma_load_3d(to, map, tid == 0 ? prod.hg * 64 : kv_col, prod.cs * TL, prod.b, bar);
      }
    } else if (tid == 0) {
      mbar_arrive_expect_tx(bar, 3 * kGatedBox);
      tma_load_3d(dst, &tm_b, prod.hg * 64, prod.cs * TL, prod.b, bar);
      tma_load_3d(dst + kGatedBox, &tm_c, prod.hg * 64, prod.cs * TL, prod.b, bar);
      tma_load_3d(dst + 2 * kGatedBox, &tm_v, prod.hg * 64, prod.cs * TL, prod.b, bar);
    }
    prod.next(ncs, hgs);
    s_prod = (s_prod + 1 == STAGES) ? 0 : s_prod + 1;
  };
  // the two logits this lane owns in a chunk (tokens 2*lane, 2*lane+1 of the warp's head)
  auto load_logits = [&](const GatedCursor& c, float (&z)[TPL]) {
    const int tok = c.cs * TL + TPL * lane;
    const long long row = static_cast<long long>(c.b) * L + tok;
    const int h = c.hg * 4 + warp;
#pragma unroll
    for (int q = 0; q < TPL; ++q) z[q] = (tok + q < L) ? __bfloat162float(p.a_logits[(row + q) * p.ld_a + h]) : 0.0f;
  };

  constexpr int AHEAD = STAGES - 2;
  for (int k = 0; k < AHEAD && k < n; ++k) issue();
  // the logits run two units ahead of the consumer: a short chunk does not hide a global load
  GatedCursor peek = cons;
  float zn[TPL], zn2[TPL];
  load_logits(peek, zn);
  peek.next(ncs, hgs);
#pragma unroll
  for (int q = 0; q < TPL; ++q) zn2[q] = 0.0f;
  if (n > 1) {
    load_logits(peek, zn2);
    peek.next(ncs, hgs);
  }

  // lane-constant addressing of this warp's [16 tokens][16 channels] block inside a box (see the header)
  const uint32_t frag_off = ((lane & 7) + 8 * (lane >> 4)) * 128 + (((2 * warp + ((lane >> 3) & 1)) ^ (lane & 7)) << 4);
  // the same block inside this warp's dense [TL][16 channels] tile of a shared key/value head (32-byte rows with
  // the 32-byte swizzle: the two 16-byte halves of rows 4..7 of every 8 rows are exchanged, which spreads the
  // eight rows of an 8x8 matrix over all banks)
  const uint32_t kv_off = SHARED ? warp * (TL * 32) + ((lane & 7) + 8 * (lane >> 4)) * 32 + ((((lane >> 3) ^ (lane >> 2)) & 1) << 4) : frag_off;
  constexpr uint32_t kKvBlock = SHARED ? 512 : 2048;  // bytes from one 16-token block to the next
  float cg = 0.0f, cg8 = 0.0f;
  int s = 0;
  uint32_t phase = 0;
  bool failed = false;
  int j = 0;
  for (; j < n; ++j) {
    if (j + AHEAD < n) {
      if (tid == 0) bulk_wait_group_read<1>();
      issue();
    }
    float l2[TPL];
#pragma unroll
    for (int q = 0; q < TPL; ++q) {
      l2[q] = logit_to_log2a(zn[q]);
      zn[q] = zn2[q];
    }
    if (j + 2 < n) {
      load_logits(peek, zn2);
      peek.next(ncs, hgs);
    }
    const bool ok = mbar_wait_bounded(bars + s * 8, phase, p.wait_limit_ns);
    if (__syncthreads_or(!ok)) {
      failed = true;
      break;
    }
    const int c0 = cons.cs * TL;
    const int left = (L - c0) >> 4;
    const int nt = left < NT ? left : NT;
    tables_from_log2<TL, false>(l2, tab, tab + TL, lane, carry_scale);
    if (cons.cs == 0 || !p.use_carry) {
      cg = cg8 = 0.0f;
    } else if (j == 0) {
      gated_halo_left(p, cons.b, cons.hg * 4 + warp, c0 - 16, lane, cg, cg8);
    }
    const float* tg = tab + tl.g;
    const float* tt = tab + 2 * tl.t;
    const uint32_t sb = base + s * SM::kStage + kv_off;
    const uint32_t sc = sb + kGatedBox;
    const uint32_t sv = base + s * SM::kStage + 2 * kGatedBox + frag_off;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      if (i < nt) {
        uint32_t bf[4], vf[4], cf[4];
        ldmatrix_x4_trans(sb + kKvBlock * i, bf[0], bf[1], bf[2], bf[3]);
        ldmatrix_x4_trans(sv + 2048 * i, vf[0], vf[1], vf[2], vf[3]);
        ldmatrix_x4_trans(sc + kKvBlock * i, cf[0], cf[1], cf[2], cf[3]);
        const uint32_t x0 = gate_pair(bf[0], vf[0]), x1 = gate_pair(bf[1], vf[1]);
        const uint32_t x2 = gate_pair(bf[2], vf[2]), x3 = gate_pair(bf[3], vf[3]);
        LmatFrag lf, lo;
        build_lmat_split(tg, tt, 16 * i, tl, lf, lo);
        float v0[4], v1[4];
        mma_16816(v0, x0, x1, x0, x1, lf.b00, lo.b00);  // hi and lo term of the 8-token product in one k = 16 instruction
        mma_16816(v1, x0, x1, x2, x3, lf.b10, lf.b11);
        mma_16816_acc(v1, x0, x1, x2, x3, lo.b10, lo.b11);
        const float2 Pa = *reinterpret_cast<const float2*>(tt + TL + 16 * i);
        const float2 Pb = *reinterpret_cast<const float2*>(tt + TL + 16 * i + 8);
        // y = v + P * carry, then out = y * C + V in the accumulator layout
        const float y00 = fmaf(Pa.x, cg, v0[0]), y01 = fmaf(Pa.y, cg, v0[1]);
        const float y02 = fmaf(Pa.x, cg8, v0[2]), y03 = fmaf(Pa.y, cg8, v0[3]);
        const float y10 = fmaf(Pb.x, cg, v1[0]), y11 = fmaf(Pb.y, cg, v1[1]);
        const float y12 = fmaf(Pb.x, cg8, v1[2]), y13 = fmaf(Pb.y, cg8, v1[3]);
        cg = __shfl_sync(0xffffffffu, v1[1], lane | 3);
        cg8 = __shfl_sync(0xffffffffu, v1[3], lane | 3);
        const uint32_t o0 = pack_bf16x2(fmaf(y00, bf16_lo(cf[0]), bf16_lo(vf[0])), fmaf(y01, bf16_hi(cf[0]), bf16_hi(vf[0])));
        const uint32_t o1 = pack_bf16x2(fmaf(y02, bf16_lo(cf[1]), bf16_lo(vf[1])), fmaf(y03, bf16_hi(cf[1]), bf16_hi(vf[1])));
        const uint32_t o2 = pack_bf16x2(fmaf(y10, bf16_lo(cf[2]), bf16_lo(vf[2])), fmaf(y11, bf16_hi(cf[2]), bf16_hi(vf[2])));
        const uint32_t o3 = pack_bf16x2(fmaf(y12, bf16_lo(cf[3]), bf16_lo(vf[3])), fmaf(y13, bf16_hi(cf[3]), bf16_hi(vf[3])));
        __syncwarp();  // every lane has its V fragment before the block is overwritten
        stmatrix_x4_trans(sv + 2048 * i, o0, o1, o2, o3);
      }
    }
    fence_proxy_async_smem();
    __syncthreads();  // all four heads of the box are in place (and nobody still reads this stage's tables)
    if (tid == 0) {
      tma_store_3d(&tm_out, cons.hg * 64, c0, cons.b, base + s * SM::kStage + 2 * kGatedBox);
      bulk_commit_group();
    }
    cons.next(ncs, hgs);
    if (++s == STAGES) {
      s = 0;
      phase ^= 1u;
    }
  }
  if (failed) {
    if (tid == 0) report_error(1u, warp, j);
    for (int k = j; k < n && k <= j + AHEAD; ++k) {  // let the loads in flight land before the CTA leaves
      mbar_wait_bounded(bars + s * 8, phase, p.wait_limit_ns);
      if (++s == STAGES) {
        s = 0;
        phase ^= 1u;
      }
    }
  }
  if (tid == 0) bulk_wait_group<0>();
}

}  // namespace btp
