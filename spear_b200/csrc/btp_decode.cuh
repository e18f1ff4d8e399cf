// Streaming (serving) side of the block two-pass recurrence: one decode step and the prefill hand-off state.
//
// Both kernels are tiny, launch-latency-bound elementwise work on [B*H, 16] tensors; what they buy is ONE launch
// where a tensor-op formulation (spear/nn/phalanx/inference.py:177-266 and 333-358 in the reference) needs a
// dozen for a step and two Python loops of up to 16 iterations each for the state.  Arithmetic is fp32 whatever
// the storage type; results are rounded once, on the store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace btp {

struct DecodeParams {
  const void* a;       // [n_heads]      gate of this token (log gate if a_log)
  const void* x;       // [n_heads, 16]  driving term
  const void* c;       // [n_heads, 16]
  const void* v;       // [n_heads, 16]
  void* y;             // [n_heads, 16]
  const void* h_in;    // [n_heads, 16]  block-local accumulator
  const void* r_in;    // [n_heads]      running gate product of the block (log of it if r_log); NULL = empty block
  const void* cprev;   // [n_heads, 16]  frozen last local value of the previous block
  void* h_out;         // [n_heads, 16]
  void* r_out;         // [n_heads]
  void* cprev_out;     // [n_heads, 16]  written only when the block completes (may be NULL otherwise)
  long long n_heads;
  int a_log;
  int r_log;
  int block_done;
};

template <class T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const void* base, long long i, float (&f)[4]) {
    const float4 q = reinterpret_cast<const float4*>(base)[i];
    f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
  }
  static __device__ __forceinline__ void store(void* base, long long i, const float (&f)[4]) {
    reinterpret_cast<float4*>(base)[i] = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const void* base, long long i, float (&f)[4]) {
    const uint2 q = reinterpret_cast<const uint2*>(base)[i];
    f[0] = __uint_as_float(q.x << 16); f[1] = __uint_as_float(q.x & 0xffff0000u);
    f[2] = __uint_as_float(q.y << 16); f[3] = __uint_as_float(q.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(void* base, long long i, const float (&f)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(f[2], f[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned*>(&lo);
    q.y = *reinterpret_cast<const unsigned*>(&hi);
    reinterpret_cast<uint2*>(base)[i] = q;
  }
};

template <class T>
__device__ __forceinline__ float load_scalar(const void* base, long long i);
template <>
__device__ __forceinline__ float load_scalar<float>(const void* base, long long i) {
  return reinterpret_cast<const float*>(base)[i];
}
template <>
__device__ __forceinline__ float load_scalar<__nv_bfloat16>(const void* base, long long i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}
template <class T>
__device__ __forceinline__ void store_scalar(void* base, long long i, float f);
template <>
__device__ __forceinline__ void store_scalar<float>(void* base, long long i, float f) {
  reinterpret_cast<float*>(base)[i] = f;
}
template <>
__device__ __forceinline__ void store_scalar<__nv_bfloat16>(void* base, long long i, float f) {
  reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(f);
}

// smallest positive normal number of the gate's storage type (the clamp of inference.py:221-223)
template <class TA>
__device__ __forceinline__ float tiny_of() { return 1.17549435e-38f; }  // the same for float and bfloat16

// One thread per 4 channels of one head.  T: storage of x, c, v, y and the two [.,16] states.  TA: gate and r.
template <class T, class TA>
__global__ void __launch_bounds__(256) btp_decode_step_kernel(const DecodeParams p) {
  const long long q = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;  // quad index
  if (q >= p.n_heads * 4) return;
  const long long head = q >> 2;
  const float a_in = load_scalar<TA>(p.a, head);
  const float a = p.a_log ? __expf(a_in) : a_in;
  float r, r_state;
  if (p.r_log) {
    const float prev = p.r_in ? load_scalar<TA>(p.r_in, head) : 0.0f;
    r_state = prev + __logf(fmaxf(a, tiny_of<TA>()));
    r = __expf(r_state);
  } else {
    const float prev = p.r_in ? load_scalar<TA>(p.r_in, head) : 1.0f;
    r = a * prev;
    r_state = r;
  }
  float h[4], x[4], c[4], v[4], cp[4], y[4];
  Vec4<T>::load(p.h_in, q, h);
  Vec4<T>::load(p.x, q, x);
  Vec4<T>::load(p.c, q, c);
  Vec4<T>::load(p.v, q, v);
  Vec4<T>::load(p.cprev, q, cp);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = fmaf(a, h[i], x[i]);
    y[i] = fmaf(fmaf(r, cp[i], h[i]), c[i], v[i]);
  }
  Vec4<T>::store(p.y, q, y);
  if (p.block_done) {  // freeze this block's last local value, start the next block empty
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    Vec4<T>::store(p.cprev_out, q, h);
    Vec4<T>::store(p.h_out, q, zero);
    if ((q & 3) == 0) store_scalar<TA>(p.r_out, head, p.r_log ? 0.0f : 1.0f);
  } else {
    Vec4<T>::store(p.h_out, q, h);
    if ((q & 3) == 0) store_scalar<TA>(p.r_out, head, r_state);
  }
}

struct PrefillStateParams {
  const void* a;   // [n_heads, L]       gates (log gates if a_log)
  const void* x;   // [n_heads, 16, L]   driving term
  void* h_loc;     // [n_heads, 16]
  void* r_pref;    // [n_heads]
  void* cprev;     // [n_heads, 16]
  long long n_heads;
  int L;
  int a_log;
};

// State after a prompt of L tokens (any L >= 1): zero-initialised scans over the last, possibly partial, block
// and over the complete block before it.  One thread per (head, channel); at most 32 steps.
template <class T, class TA>
__global__ void __launch_bounds__(256) btp_prefill_state_kernel(const PrefillStateParams p) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= p.n_heads * 16) return;
  const long long head = idx >> 4;
  const int L = p.L;
  const int tail_i = (L - 1) & 15;
  const int s_last = (L - 1) & ~15;
  const long long arow = head * L;
  const long long xrow = idx * L;
  float h = 0.0f, r = 1.0f;
  for (int t = s_last; t < L; ++t) {
    const float g = load_scalar<TA>(p.a, arow + t);
    const float a = p.a_log ? __expf(g) : g;
    h = fmaf(a, h, load_scalar<T>(p.x, xrow + t));
    r *= a;
  }
  float cp = 0.0f;
  if (tail_i == 15) {
    // The prompt ends on a block boundary.  The reference hands the finished block's last local value on in
    // BOTH fields and only resets the gate product (inference.py:339-342); kept as it is for identical results.
    cp = h;
    r = 1.0f;
  } else if (s_last >= 16) {
    for (int t = s_last - 16; t < s_last; ++t) {
      const float g = load_scalar<TA>(p.a, arow + t);
      const float a = p.a_log ? __expf(g) : g;
      cp = fmaf(a, cp, load_scalar<T>(p.x, xrow + t));
    }
  }
  store_scalar<T>(p.h_loc, idx, h);
  store_scalar<T>(p.cprev, idx, cp);
  if ((idx & 15) == 0) store_scalar<TA>(p.r_pref, head, r);
}

}  // namespace btp
