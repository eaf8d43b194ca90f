// What an attention mixer may do to its queries and keys between the input projection and the cache, and to its result
// before the output projection.
//
// tlc_qk_rotate_norm works on the 32-bit projection in place, a warp per (row, head), query heads and key heads alike:
// it turns the pairs of the first `rot` dimensions of a head by angle = position * inv_freq[i] (pairs (2i, 2i+1) with
// interleaved != 0, else (i, i + rot/2); dimensions past `rot` pass unchanged) and then, with norm_eps >= 0, scales the
// head to unit root mean square over its `dim` dimensions, x / sqrt(mean(x^2) + eps), without a weight.  With q_w and k_w
// (weights [dim], one for all query heads and one for all key heads) every head is first normed BEFORE the rotation,
// x / sqrt(mean(x^2) + pre_eps) * w; `amplitude` multiplies every cosine and sine (1: a plain rotation).  Heads may lie
// `stride` >= dim values apart (a mixer whose values are wider than its keys pads the heads; the padding stays zero).
// Everything is 32-bit; the kernels that store keys and values then need not rotate.
//
// tlc_gate_mul multiplies a [T, n] activation in place by sigmoid (or SiLU) of a column range of the 32-bit projection:
// an output gate that reads the same input as the projections.
#include "common.cuh"

#define QK_MAXV 8     // a head of at most 32 * QK_MAXV dimensions

__global__ void __launch_bounds__(128)
qk_rotate_norm_kernel(float* __restrict__ qkv, int ld, int q_off, int k_off, int H, int KV, int stride, int dim,
                      const float* __restrict__ inv_freq, int rot, int interleaved, float norm_eps,
                      const int* __restrict__ positions, int T, const float* __restrict__ q_w, const float* __restrict__ k_w,
                      float pre_eps, float amplitude) {
  tlc_pdl(qkv);
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int units = H + KV;
  if (w >= T * units) return;
  const int t = w / units, u = w - t * units;
  float* x = qkv + (size_t)t * ld + (u < H ? q_off + u * stride : k_off + (u - H) * stride);
  const float fpos = (float)positions[t];
  const int half = rot >> 1;
  // a weighted RMS norm of the head BEFORE the rotation (pre_w): x <- x / sqrt(mean(x^2) + pre_eps) * pre_w
  const float* pre_w = u < H ? q_w : k_w;
  float pre = 1.0f;
  if (pre_w) {
    float p2 = 0.f;
    for (int d = lane; d < dim; d += 32) { const float v = x[d]; p2 += v * v; }
    pre = 1.0f / sqrtf(warp_sum(p2) / (float)dim + pre_eps);
  }
  float ss = 0.f;
  for (int p = lane; p < half; p += 32) {
    const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
    float sn, cs;
    sincosf(fpos * inv_freq[p], &sn, &cs);
    sn *= amplitude;
    cs *= amplitude;
    float a = x[ia], b = x[ib];
    if (pre_w) { a = a * pre * pre_w[ia]; b = b * pre * pre_w[ib]; }
    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
    x[ia] = ra;
    x[ib] = rb;
    ss += ra * ra + rb * rb;
  }
  if (pre_w)
    for (int d = rot + lane; d < dim; d += 32) x[d] = x[d] * pre * pre_w[d];
  if (norm_eps < 0.f) return;
  for (int d = rot + lane; d < dim; d += 32) { const float v = x[d]; ss += v * v; }
  ss = warp_sum(ss);
  const float s = 1.0f / sqrtf(ss / (float)dim + norm_eps);
  __syncwarp();
  for (int d = lane; d < dim; d += 32) x[d] *= s;
}

extern "C" int tlc_qk_rotate_norm(float* qkv, int ld, int q_off, int k_off, int H, int KV, int stride, int dim,
                                  const float* inv_freq, int rot, int interleaved, float norm_eps, const int* positions, int T,
                                  const float* q_w, const float* k_w, float pre_eps, float amplitude, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(dim >= 1 && dim <= stride && rot >= 0 && rot % 2 == 0 && rot <= dim, "qk_rotate_norm: %d rotated of %d dimensions, heads %d apart",
              rot, dim, stride);
  TLC_REQUIRE((q_w == nullptr) == (k_w == nullptr), "qk_rotate_norm: the weights of the norm before the rotation come together");
  const long long warps = (long long)T * (H + KV);
  tlc_launch(qk_rotate_norm_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, qkv, ld, q_off, k_off, H, KV, stride, dim,
             inv_freq, rot, interleaved, norm_eps, positions, T, q_w, k_w, pre_eps, amplitude);
  TLC_CHECK_LAUNCH("qk_rotate_norm");
  return 0;
}

// Four neighbouring elements a thread (n a multiple of 4, rows that start on 16-byte boundaries of the gate and 8-byte
// (bfloat16) or 16-byte (float) boundaries of x), else one.
template <typename TX, bool QUICK, int VEC>
__global__ void __launch_bounds__(256)
gate_mul_kernel(TX* __restrict__ x, int ldx, const float* __restrict__ gate, int ldg, int n, int T, int act) {
  tlc_pdl(x, gate);
  const int per_row = n / VEC;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * per_row) return;
  const int t = (int)(i / per_row), c = (int)(i - (long long)t * per_row) * VEC;
  float g[VEC], v[VEC];
  TX* p = x + (size_t)t * ldx + c;
  if (VEC == 4) {
    const float4 g4 = *reinterpret_cast<const float4*>(gate + (size_t)t * ldg + c);
    g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[VEC - 1] = g4.w;
    if (sizeof(TX) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[VEC - 1] = __high2float(hi);
    } else {
      const float4 x4 = *reinterpret_cast<const float4*>(p);
      v[0] = x4.x; v[1] = x4.y; v[2] = x4.z; v[VEC - 1] = x4.w;
    }
  } else {
    g[0] = gate[(size_t)t * ldg + c];
    v[0] = to_f32(*p);
  }
#pragma unroll
  for (int e = 0; e < VEC; e++) {
    const float s = QUICK ? __fdividef(1.0f, 1.0f + __expf(-g[e])) : 1.0f / (1.0f + expf(-g[e]));
    v[e] *= act == 1 ? g[e] * s : s;
  }
  if (VEC == 4) {
    if (sizeof(TX) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[VEC - 1]);
      uint2 raw;
      raw.x = *reinterpret_cast<unsigned*>(&lo);
      raw.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(p) = raw;
    } else {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[VEC - 1]);
    }
  } else {
    *p = from_f32<TX>(v[0]);
  }
}

// x[t, c] *= sigmoid(gate[t, c]) (act 0) or silu(gate[t, c]) (act 1); x [T, n] of `dtype` with row stride ldx, gate float
// with row stride ldg.
extern "C" int tlc_gate_mul(void* x, int dtype, int ldx, const float* gate, int ldg, int n, int T, int act, cudaStream_t stream) {
  if (T == 0 || n == 0) return 0;
  TLC_REQUIRE(act == 0 || act == 1, "gate_mul: unknown gate %d", act);
  const size_t esz = dtype == TLC_BF16 ? 2 : 4;
  const bool vec = n % 4 == 0 && ldg % 4 == 0 && (uintptr_t)gate % 16 == 0 && (ldx * esz) % (4 * esz) == 0 && (uintptr_t)x % (4 * esz) == 0;
  const long long total = (long long)T * (vec ? n / 4 : n);
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype != TLC_BF16 && dtype != TLC_F32) return tlc_fail(-1, "gate_mul: unknown dtype code %d", dtype);
  if (dtype == TLC_BF16) {
    if (vec) tlc_launch(gate_mul_kernel<__nv_bfloat16, true, 4>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, ldx, gate, ldg, n, T, act);
    else tlc_launch(gate_mul_kernel<__nv_bfloat16, true, 1>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, ldx, gate, ldg, n, T, act);
  } else {
    if (vec) tlc_launch(gate_mul_kernel<float, false, 4>, grid, dim3(256), 0, stream, (float*)x, ldx, gate, ldg, n, T, act);
    else tlc_launch(gate_mul_kernel<float, false, 1>, grid, dim3(256), 0, stream, (float*)x, ldx, gate, ldg, n, T, act);
  }
  TLC_CHECK_LAUNCH("gate_mul");
  return 0;
}

// ---- queries and keys normed over their whole width -----------------------------------------------------------------
// In place on the 32-bit projection: the q_n query columns from q_off (all heads together) are divided by their root mean
// square and multiplied by qw [q_n], the k_n key columns from k_off likewise with kw; before any rotation.  One block per row.
__global__ void __launch_bounds__(256)
qk_whole_norm_kernel(float* qkv, int ld, int q_off, int q_n, const float* __restrict__ qw, int k_off, int k_n,
                     const float* __restrict__ kw, float eps) {
  tlc_pdl(qkv);
  __shared__ float red[33];
  float* row = qkv + (size_t)blockIdx.x * ld;
  for (int which = 0; which < 2; which++) {
    float* x = row + (which ? k_off : q_off);
    const int n = which ? k_n : q_n;
    const float* w = which ? kw : qw;
    float ss = 0.f;
    for (int d = threadIdx.x; d < n; d += blockDim.x) { const float v = x[d]; ss += v * v; }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    for (int d = threadIdx.x; d < n; d += blockDim.x) x[d] = x[d] * s * w[d];
  }
}
extern "C" int tlc_qk_whole_norm(float* qkv, int ld, int q_off, int q_n, const float* qw, int k_off, int k_n, const float* kw, float eps,
                                 int T, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(q_n >= 1 && k_n >= 1, "qk_whole_norm: %d query and %d key columns", q_n, k_n);
  tlc_launch(qk_whole_norm_kernel, dim3(T), dim3(256), 0, stream, qkv, ld, q_off, q_n, qw, k_off, k_n, kw, eps);
  TLC_CHECK_LAUNCH("qk_whole_norm");
  return 0;
}
