// A time-mixing layer with a decaying matrix state per head and a bonus for the current token:
//
//   o_t = (S + diag(u) k_t v_t^T)^T r_t          S <- diag(w_t) S + k_t v_t^T          w_t = exp(-exp(a_t))
//
// S [d, d] per head (rows: key channels, columns: value channels), 32-bit, carried per sequence; u [H, d] learned; r, k, v
// and the decay's logarithm a arrive as columns of 32-bit projections.  Every projection of such a layer reads a mix of
// its own of the token's input and the previous token's: m_s[t] = x[t] + (x[t-1] - x[t]) * mu_s (tlc_shift_mix), the
// previous token's row being part of the sequence's state as well.
//
// The scan (tlc_wkv_scan): column j of S depends on column j alone.  A block owns 32 columns of one (sequence, head); a
// column's d rows are split among R neighbouring lanes (R = 1, 2, 4 or 8, at most 32 rows a lane, in registers), which
// join their partial read-outs by shuffles.  The bonus term is the same for every column, v_j * sum_i r_i u_i k_i, so a
// lane adds its rows' share of that sum on the way.  Tokens are staged through shared memory 16 at a time (the decay's
// two exponentials are taken there, once per element); the state is read once and written once per step.
#include "common.cuh"

#define WKV_COLS 32
#define WKV_TOK 16
#define WKV_RPL 32           // rows of a column that one lane holds at most

// out[t, s, :] = x[t] + (prev - x[t]) * mu[s], prev the row above or the slot's kept row (zeros at position 0); the block of
// a sequence's first row of the step, the only one that reads the slot, afterwards leaves the sequence's last row there.
template <typename TO>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const float* __restrict__ x, const float* __restrict__ mu, int n_mix, int D, const int* __restrict__ row_seq,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots, const int* __restrict__ start_pos, float* state,
                 TO* __restrict__ out) {
  tlc_pdl(x, state, out);
  const int t = blockIdx.x, b = row_seq[t];
  const int first = cu_seqlens[b], last = cu_seqlens[b + 1] - 1;
  const float* xr = x + (size_t)t * D;
  float* st = state + (size_t)slots[b] * D;
  const bool from_state = t == first, fresh = start_pos[b] == 0;
  const float* xl = x + (size_t)last * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float cur = xr[d];
    const float prev = from_state ? (fresh ? 0.f : st[d]) : xr[d - D];
    const float diff = prev - cur;
    for (int s = 0; s < n_mix; s++)
      out[((size_t)t * n_mix + s) * D + d] = from_f32<TO>(fmaf(diff, mu[(size_t)s * D + d], cur));
    if (from_state) st[d] = xl[d];           // (read above by this thread)
  }
}

extern "C" int tlc_shift_mix(const float* x, const float* mu, int n_mix, int T, int D, const int* row_seq, const int* cu_seqlens,
                             const int* slots, const int* start_pos, float* state, void* out, int out_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(n_mix >= 1, "shift_mix: %d mixes", n_mix);
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(shift_mix_kernel<TO>, dim3(T), dim3(256), 0, stream, x, mu, n_mix, D, row_seq, cu_seqlens,
                                               slots, start_pos, state, (TO*)out));
  TLC_CHECK_LAUNCH("shift_mix");
  return 0;
}

template <int R>
__global__ void __launch_bounds__(WKV_COLS * R)
wkv_scan_kernel(const float* __restrict__ rkv, int ld, int r_off, int k_off, int v_off, const float* __restrict__ decay_log, int ld_w,
                const float* __restrict__ bonus, float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                const int* __restrict__ start_pos, int H, int d, float* __restrict__ out, int out_ld) {
  tlc_pdl(rkv, decay_log, state, out);
  extern __shared__ float wkv_sh[];
  float* rs = wkv_sh;                         // [WKV_TOK][d] each
  float* ks = rs + (size_t)WKV_TOK * d;
  float* ws = ks + (size_t)WKV_TOK * d;
  float* vs = ws + (size_t)WKV_TOK * d;       // [WKV_TOK][WKV_COLS]
  float* us = vs + (size_t)WKV_TOK * WKV_COLS; // [d]
  const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * WKV_COLS;
  const int tid = threadIdx.x, nt = WKV_COLS * R;
  const int part = tid % R, jj = tid / R, j = j0 + jj;
  const int rows = (d + R - 1) / R;           // rows of a column a lane holds (<= WKV_RPL)
  const int i0 = part * rows;
  const bool col = j < d;
  float S[WKV_RPL];
  float* sp = state + (((size_t)slots[b] * H + h) * d) * d;
  const bool fresh = start_pos[b] == 0;
#pragma unroll
  for (int i = 0; i < WKV_RPL; i++) {
    const int row = i0 + i;
    S[i] = (!fresh && col && i < rows && row < d) ? sp[(size_t)row * d + j] : 0.f;
  }
  for (int i = tid; i < d; i += nt) us[i] = bonus[(size_t)h * d + i];
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  for (int tb = t0; tb < t1; tb += WKV_TOK) {
    const int n = min(WKV_TOK, t1 - tb);
    __syncthreads();                          // the tile before is walked
    for (int idx = tid; idx < n * d; idx += nt) {
      const int tt = idx / d, i = idx % d;
      const float* pr = rkv + (size_t)(tb + tt) * ld + (size_t)h * d + i;
      rs[idx] = pr[r_off];
      ks[idx] = pr[k_off];
      ws[idx] = expf(-expf(decay_log[(size_t)(tb + tt) * ld_w + (size_t)h * d + i]));
    }
    for (int idx = tid; idx < n * WKV_COLS; idx += nt) {
      const int tt = idx / WKV_COLS, c = idx % WKV_COLS;
      vs[idx] = j0 + c < d ? rkv[(size_t)(tb + tt) * ld + v_off + (size_t)h * d + j0 + c] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < n; tt++) {
      const float* r = rs + (size_t)tt * d + i0;
      const float* k = ks + (size_t)tt * d + i0;
      const float* w = ws + (size_t)tt * d + i0;
      const float v = vs[tt * WKV_COLS + jj];
      float read = 0.f, extra = 0.f;
#pragma unroll
      for (int i = 0; i < WKV_RPL; i++) {
        if (i < rows && i0 + i < d) {
          const float ri = r[i], ki = k[i];
          read = fmaf(ri, S[i], read);
          extra = fmaf(ri * us[i0 + i], ki, extra);
          S[i] = fmaf(w[i], S[i], ki * v);
        }
      }
      float o = fmaf(extra, v, read);
#pragma unroll
      for (int s = 1; s < R; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (part == 0 && col) out[(size_t)(tb + tt) * out_ld + (size_t)h * d + j] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < WKV_RPL; i++) {
    const int row = i0 + i;
    if (col && i < rows && row < d) sp[(size_t)row * d + j] = S[i];
  }
}

extern "C" int tlc_wkv_scan(const float* rkv, int ld, int r_off, int k_off, int v_off, const float* decay_log, int ld_w,
                            const float* bonus, float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B,
                            int H, int d, float* out, int out_ld, cudaStream_t stream) {
  if (B == 0 || H == 0) return 0;
  TLC_REQUIRE(d >= 1 && d <= 8 * WKV_RPL, "wkv_scan: heads of %d channels are outside what the kernel is built for (1..%d)", d, 8 * WKV_RPL);
  TLC_REQUIRE(H <= 65535, "wkv_scan: too many heads (%d)", H);
  const int need = (d + WKV_RPL - 1) / WKV_RPL;
  const int R = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  const size_t smem = ((size_t)3 * WKV_TOK * d + (size_t)WKV_TOK * WKV_COLS + d) * sizeof(float);
  dim3 grid(B, H, (d + WKV_COLS - 1) / WKV_COLS);
  // (more than 48 KB of dynamic shared memory, which heads of more than 224 channels need, must be asked for)
#define WKV_LAUNCH(RR)                                                                                                        \
  do {                                                                                                                        \
    if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    tlc_launch(wkv_scan_kernel<RR>, grid, dim3(WKV_COLS * RR), smem, stream, rkv, ld, r_off, k_off, v_off, decay_log, ld_w,       \
               bonus, state, cu_seqlens, slots, start_pos, H, d, out, out_ld);                                                  \
  } while (0)
  if (R == 1) WKV_LAUNCH(1);
  else if (R == 2) WKV_LAUNCH(2);
  else if (R == 4) WKV_LAUNCH(4);
  else WKV_LAUNCH(8);
#undef WKV_LAUNCH
  TLC_CHECK_LAUNCH("wkv_scan");
  return 0;
}
