// Layer norm of 32-bit rows, a learned row added to every row, and the join of two attention maps.
//
// tlc_layernorm: out[r] = (x - mean(x)) / sqrt(var(x) + eps) * w with var the mean of the squared deviations; no bias.
// A layer whose two sublayers each norm the SAME rows with a weight of their own gets both results from one pass:
// the statistics are computed once, out2 = the same normed row times w2.  The row stays in registers between the
// mean, the variance and the scaling (a second pass over the deviations, not E[x^2] - mean^2, which cancels).
//
// tlc_add_row: x[t, :] += v[:] (a learned vector that marks the pass of a repeated range of layers).
//
// tlc_difference_join: two attention maps per head over the same values, a1 and a2 [vd]:
//   o = a1 - lambda a2;   o <- o / sqrt(mean(o^2) + eps) * out_scale
// a warp per (row, head); the maps of query head h lie at virtual heads first(h) and first(h) + step of the input.
#include "common.cuh"

#define LN_MAX_PER_THREAD 16      // a row of up to 256 * 16 values stays in registers

template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, int x_ld, const int* __restrict__ rows, const float* __restrict__ w1,
                 const float* __restrict__ w2, float eps, int D, TO* __restrict__ out1, TO* __restrict__ out2) {
  tlc_pdl(x, rows, out1, out2);
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * x_ld;
  if (D <= 256 * LN_MAX_PER_THREAD) {
    float v[LN_MAX_PER_THREAD];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < LN_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      v[i] = d < D ? xr[d] : 0.f;
      s += v[i];
    }
    const float mean = block_sum(s, red) / (float)D;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < LN_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      v[i] = d < D ? v[i] - mean : 0.f;
      ss += v[i] * v[i];
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
#pragma unroll
    for (int i = 0; i < LN_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      if (d < D) {
        const float n = v[i] * inv;
        out1[(size_t)r * D + d] = from_f32<TO>(n * w1[d]);
        if (out2) out2[(size_t)r * D + d] = from_f32<TO>(n * w2[d]);
      }
    }
    return;
  }
  float s = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) s += xr[d];
  const float mean = block_sum(s, red) / (float)D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = xr[d] - mean; ss += c * c; }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float n = (xr[d] - mean) * inv;
    out1[(size_t)r * D + d] = from_f32<TO>(n * w1[d]);
    if (out2) out2[(size_t)r * D + d] = from_f32<TO>(n * w2[d]);
  }
}

// Rows whose width is a multiple of 4 (up to 4096 float4): NT threads take PT float4 each, 16-byte loads and stores.
// NT and PT follow from the width and from whether the step has 512 rows or more; a prompt cut into portions may so take
// another tree for a row's sums than the whole prompt does, which moves a result by rounding only.
template <typename TO> struct LnOut4;
template <> struct LnOut4<float> {
  static __device__ __forceinline__ void put(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
};
template <> struct LnOut4<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename TO, int NT, int PT>
__global__ void __launch_bounds__(NT)
layernorm_vec_kernel(const float* __restrict__ x, int x_ld, const int* __restrict__ rows, const float* __restrict__ w1,
                     const float* __restrict__ w2, float eps, int D, TO* __restrict__ out1, TO* __restrict__ out2) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const int n4 = D >> 2, r = blockIdx.x;
  // the weights do not depend on the kernel before this one: they are fetched before the wait on it
  float4 wa[PT], wb[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wa[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w1) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    wb[i] = (w2 != nullptr && c < n4) ? __ldg(reinterpret_cast<const float4*>(w2) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(x, rows, out1, out2);
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * x_ld);
  float4 v[PT];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = block_sum(s, red) / (float)D;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4) {
      const float4 a = wa[i];
      LnOut4<TO>::put(out1 + (size_t)r * D + 4 * c, v[i].x * inv * a.x, v[i].y * inv * a.y, v[i].z * inv * a.z, v[i].w * inv * a.w);
      if (out2) {
        const float4 b = wb[i];
        LnOut4<TO>::put(out2 + (size_t)r * D + 4 * c, v[i].x * inv * b.x, v[i].y * inv * b.y, v[i].z * inv * b.z, v[i].w * inv * b.w);
      }
    }
  }
}

extern "C" int tlc_layernorm(const float* x, int x_ld, const int* rows, const float* w1, const float* w2, float eps, int R, int D,
                             void* out1, void* out2, int out_dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  TLC_REQUIRE(x_ld >= D && D >= 1, "layernorm: rows of %d values with a stride of %d", D, x_ld);
  TLC_REQUIRE((w2 == nullptr) == (out2 == nullptr), "layernorm: a second weight and a second output come together");
  const bool aligned = D % 4 == 0 && x_ld % 4 == 0 && D <= 16384 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w1 % 16) == 0 &&
                       ((uintptr_t)out1 % 16) == 0 && ((uintptr_t)w2 % 16) == 0 && ((uintptr_t)out2 % 16) == 0;
  if (aligned) {
    const int n4 = D / 4;
#define TLC_LN_LAUNCH(NT, PT)                                                                                                   \
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(layernorm_vec_kernel<TO, NT, PT>, dim3(R), dim3(NT), 0, stream, x, x_ld, rows, w1, w2, \
                                               eps, D, (TO*)out1, (TO*)out2))
    if (R >= 512) {          // many rows (prompts): fewer threads a row with up to four pieces each, more rows an SM
      if (n4 <= 128) { TLC_LN_LAUNCH(64, 2); }
      else if (n4 <= 256) { TLC_LN_LAUNCH(64, 4); }
      else if (n4 <= 512) { TLC_LN_LAUNCH(128, 4); }
      else if (n4 <= 768) { TLC_LN_LAUNCH(256, 3); }
      else if (n4 <= 1024) { TLC_LN_LAUNCH(256, 4); }
      else if (n4 <= 2048) { TLC_LN_LAUNCH(512, 4); }
      else { TLC_LN_LAUNCH(1024, 4); }
    } else {                 // few rows: a piece a thread, so that the row's loads are all in flight at once
      if (n4 <= 128) { TLC_LN_LAUNCH(128, 1); }
      else if (n4 <= 256) { TLC_LN_LAUNCH(256, 1); }
      else if (n4 <= 512) { TLC_LN_LAUNCH(512, 1); }
      else if (n4 <= 1024) { TLC_LN_LAUNCH(1024, 1); }
      else if (n4 <= 2048) { TLC_LN_LAUNCH(1024, 2); }
      else { TLC_LN_LAUNCH(1024, 4); }
    }
#undef TLC_LN_LAUNCH
    TLC_CHECK_LAUNCH("layernorm");
    return 0;
  }
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(layernorm_kernel<TO>, dim3(R), dim3(256), 0, stream, x, x_ld, rows, w1, w2, eps, D,
                                               (TO*)out1, (TO*)out2));
  TLC_CHECK_LAUNCH("layernorm");
  return 0;
}

// ---- x[t, :] += v ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) add_row_kernel(float* __restrict__ x, const float* __restrict__ v, int D, size_t total) {
  tlc_pdl(x);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] += v[i % D];
}
__global__ void __launch_bounds__(256) add_row4_kernel(float4* __restrict__ x, const float4* __restrict__ v, int D4, size_t total4) {
  tlc_pdl(x);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  float4 a = x[i];
  const float4 b = __ldg(v + i % D4);
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  x[i] = a;
}
extern "C" int tlc_add_row(float* x, const float* v, int T, int D, cudaStream_t stream) {
  const size_t total = (size_t)T * D;
  if (total == 0) return 0;
  if (D % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)v % 16) == 0)
    tlc_launch(add_row4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (float4*)x, (const float4*)v, D / 4, total / 4);
  else
    tlc_launch(add_row_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, v, D, total);
  TLC_CHECK_LAUNCH("add_row");
  return 0;
}

// ---- the join of two attention maps ----------------------------------------------------------------------------------------
// att [T, ld_in]: virtual head j's result (hd values, the first vd in use) at column j * hd.  Query head h of group
// g = h / per_group has its first map at virtual head (2 g) * per_group + (h - g * per_group) and its second per_group heads
// further on.  out [T, ld_out]: head h at column h * hd_out, vd values (the rest of a padded head is left as it is).
#define DJ_MAXV 8
template <typename T>
__global__ void __launch_bounds__(128)
difference_join_kernel(const T* __restrict__ att, int ld_in, int hd, T* __restrict__ out, int ld_out, int hd_out, int H, int per_group,
                       int vd, float lambda, float eps, float out_scale, int n_rows) {
  tlc_pdl(att, out);
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= n_rows * H) return;
  const int t = w / H, h = w - t * H;
  const int g = h / per_group;
  const T* a1 = att + (size_t)t * ld_in + (size_t)(2 * g * per_group + (h - g * per_group)) * hd;
  const T* a2 = a1 + (size_t)per_group * hd;
  float o[DJ_MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < DJ_MAXV; i++) {
    const int d = lane + 32 * i;
    o[i] = d < vd ? to_f32(a1[d]) - lambda * to_f32(a2[d]) : 0.f;
    ss += o[i] * o[i];
  }
  ss = warp_sum(ss);
  const float s = out_scale / sqrtf(ss / (float)vd + eps);
  T* dst = out + (size_t)t * ld_out + (size_t)h * hd_out;
#pragma unroll
  for (int i = 0; i < DJ_MAXV; i++) {
    const int d = lane + 32 * i;
    if (d < vd) dst[d] = from_f32<T>(o[i] * s);
  }
}

extern "C" int tlc_difference_join(const void* att, int dtype, int ld_in, int hd, void* out, int ld_out, int hd_out, int T, int H,
                                   int per_group, int vd, float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(H >= 1 && per_group >= 1 && H % per_group == 0 && vd >= 1 && vd <= hd && vd <= hd_out && vd <= 32 * DJ_MAXV,
              "difference_join: %d heads in groups of %d, %d of %d values", H, per_group, vd, hd);
  const long long warps = (long long)T * H;
  TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(difference_join_kernel<TT>, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream,
                                           (const TT*)att, ld_in, hd, (TT*)out, ld_out, hd_out, H, per_group, vd, lambda, eps, out_scale, T));
  TLC_CHECK_LAUNCH("difference_join");
  return 0;
}
