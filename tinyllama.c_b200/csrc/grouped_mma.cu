// Grouped products on the tensor cores (mma.sync, bfloat16 operands, 32-bit sums): many small matrix products that
// share a shape but not their weights -- one per attention head, or one per expert over the rows routed to it.
//
// A block computes a tile of 32 (or, for groups of many rows, 64) rows x 64 columns of ONE group: two warps along the
// rows, two along the columns.
// Operand tiles of 32 K-values arrive by cp.async (three or six stages) in rows padded by 16 bytes, so that ldmatrix reads
// without bank conflicts; rows past the group's end, columns past N and K-values past K are zero-filled by the copy
// itself.  Three uses, chosen by MODE:
//   heads    out[t, h, n] = sum_k a[t, h, k] w[h, n, k]                       (group = head, rows = all T rows)
//   gate_up  act[i, f] = silu(w_i g) * (w_i u), g | u = Wgu[e] x[token(i)]     (group = expert, rows = its sorted pairs)
//   down     y[pair(i), :] = Wd[e] act[i, :]
// The expert modes read the routing that tlc_moe_route leaves on the device (order, offsets, tile_off); their grid is an
// upper bound and a block past the last tile returns.
#include "common.cuh"

#define GM_TM 32
#define GM_TN 64
#define GM_TK 32
#define GM_LD (GM_TK + 8)

__device__ __forceinline__ void gm_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void gm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void gm_ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void gm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum { GM_HEADS = 0, GM_GATE_UP = 1, GM_DOWN = 2, GM_UP = 3 };      // GM_UP: an expert without a gate, act[i, f] = f(W[e] x[token(i)])

struct GmArgs {
  const __nv_bfloat16* a;      // heads: [T, lda] with head h at h * a_hs; gate_up: x [T, lda]; down: act [pairs, K]
  const __nv_bfloat16* w;      // heads: [H, N, K]; gate_up: [E, 2N, K]; down: [E, N, K]
  void* out;                   // heads: rows of ldo, head h at h * o_hs (float or bfloat16); gate_up: act [pairs, N]
                               // bfloat16; down: y [pairs, N] float
  const int* order; const int* offsets; const int* tile_off; const float* wts;
  int lda, a_hs, ldo, o_hs, T, N, K, E, top, out_f32;
  int act, w_out;              // gate_up: the activation's code and where the pair's weight goes (moe_pair_act)
  float limit, alpha;
};

// WM: 16-row tiles a warp takes along the rows (1: a block's tile is 32 rows, 2: 64 rows, for groups with many rows).
// STAGES: operand tiles in flight.  With few rows a group the grid is a few hundred blocks that each stream a slab of
// weights: six stages keep enough bytes on their way; with many rows three.
template <int MODE, int WM> struct GmShape {
  static constexpr int NW = MODE == GM_GATE_UP ? 2 : 1;            // weight tiles per stage (gate and up)
  static constexpr int TM = GM_TM * WM;
  static constexpr int STAGES = WM == 1 ? 6 : 3;
  static constexpr size_t SMEM = (size_t)STAGES * (TM + NW * GM_TN) * GM_LD * sizeof(__nv_bfloat16);
};

template <int MODE, int WM>
__global__ void __launch_bounds__(128)
grouped_mma_kernel(GmArgs p) {
  tlc_pdl(p.a, p.out, p.order, p.offsets, p.tile_off, p.wts);
  constexpr int NW = GmShape<MODE, WM>::NW, TM = GmShape<MODE, WM>::TM, STAGES = GmShape<MODE, WM>::STAGES;
  extern __shared__ __align__(16) unsigned char gm_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gm_smem);                  // [STAGES][TM][GM_LD]
  __nv_bfloat16* Ws = As + (size_t)STAGES * TM * GM_LD;                           // [STAGES][NW][GM_TN][GM_LD]
  __shared__ int src_row[TM];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q4 = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;
  const int n0 = blockIdx.y * GM_TN;
  int group, row0, rows;
  if (MODE == GM_HEADS) {
    group = blockIdx.z;
    row0 = blockIdx.x * TM;
    rows = min(TM, p.T - row0);
  } else {
    const int tile = blockIdx.x;
    if (tile >= p.tile_off[p.E]) return;
    int lo = 0, hi = p.E - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.tile_off[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    group = lo;
    row0 = p.offsets[lo] + (tile - p.tile_off[lo]) * TM;
    rows = min(TM, p.offsets[lo + 1] - row0);
    if (tid < TM) src_row[tid] = tid < rows ? p.order[row0 + tid] : 0;
    __syncthreads();
  }
  const int K = p.K, N = p.N;
  // this thread's copies: WM 16-byte pieces of the A tile, two of every weight tile
  const int ac = (tid & 3) * 8;
  const __nv_bfloat16* a_src[WM];
  bool a_ok[WM];
#pragma unroll
  for (int j = 0; j < WM; j++) {
    const int ar = (tid >> 2) + j * 32;
    if (MODE == GM_HEADS) a_src[j] = p.a + (size_t)group * p.a_hs + (size_t)min(row0 + ar, p.T - 1) * p.lda;
    else if (MODE == GM_GATE_UP || MODE == GM_UP) a_src[j] = p.a + (size_t)(src_row[ar] / p.top) * p.lda;
    else a_src[j] = p.a + (size_t)(row0 + min(ar, rows - 1)) * K;
    a_ok[j] = ar < rows;
  }
  const __nv_bfloat16* wg = p.w + (size_t)group * (MODE == GM_GATE_UP ? 2 : 1) * N * K;
  const __nv_bfloat16* w_src[NW][2];
  bool w_ok[2];
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const int wr = (tid >> 2) + j * 32;
    w_ok[j] = n0 + wr < N;
    const int n = min(n0 + wr, N - 1);
#pragma unroll
    for (int u = 0; u < NW; u++) w_src[u][j] = wg + ((size_t)u * N + n) * K;
  }
  const uint32_t as_u = (uint32_t)__cvta_generic_to_shared(As), ws_u = (uint32_t)__cvta_generic_to_shared(Ws);
  auto load = [&](int k0, int buf) {
    const int k = k0 + ac;
    const bool k_ok = k < K;
    const int kk = k_ok ? k : 0;
#pragma unroll
    for (int j = 0; j < WM; j++)
      gm_cp16(as_u + (uint32_t)((buf * TM + (tid >> 2) + j * 32) * GM_LD + ac) * 2, a_src[j] + kk, (a_ok[j] && k_ok) ? 16 : 0);
#pragma unroll
    for (int u = 0; u < NW; u++)
#pragma unroll
      for (int j = 0; j < 2; j++)
        gm_cp16(ws_u + (uint32_t)(((buf * NW + u) * GM_TN + (tid >> 2) + j * 32) * GM_LD + ac) * 2, w_src[u][j] + kk,
                (w_ok[j] && k_ok) ? 16 : 0);
  };
  float acc[NW][WM][4][4];
#pragma unroll
  for (int u = 0; u < NW; u++)
#pragma unroll
    for (int i = 0; i < WM; i++)
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[u][i][j][e] = 0.f;
  const int n_k = (K + GM_TK - 1) / GM_TK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; st++) {
    if (st < n_k) load(st * GM_TK, st);
    gm_commit();
  }
  for (int ks = 0; ks < n_k; ks++) {
    const int buf = ks % STAGES;
    gm_wait<STAGES - 2>();                     // the tile of this step has landed
    __syncthreads();                           // ... for every thread, and every warp is done with the step before
    const int nxt = ks + STAGES - 1;           // its buffer takes the tile STAGES - 1 steps ahead
    if (nxt < n_k) load(nxt * GM_TK, nxt % STAGES);
    gm_commit();
#pragma unroll
    for (int k16 = 0; k16 < GM_TK; k16 += 16) {
      uint32_t af[WM][4];
#pragma unroll
      for (int i = 0; i < WM; i++)
        gm_ldsm4(af[i][0], af[i][1], af[i][2], af[i][3],
                 as_u + (uint32_t)((buf * TM + (wm * WM + i) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * GM_LD + k16 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int u = 0; u < NW; u++)
#pragma unroll
        for (int jp = 0; jp < 2; jp++) {
          uint32_t b0, b1, b2, b3;
          gm_ldsm4(b0, b1, b2, b3, ws_u + (uint32_t)(((buf * NW + u) * GM_TN + wn * 32 + jp * 16 + (lane & 7) + (lane >> 4) * 8) * GM_LD + k16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
          for (int i = 0; i < WM; i++) {
            gm_mma(acc[u][i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], b0, b1);
            gm_mma(acc[u][i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], b2, b3);
          }
        }
    }
  }
  gm_wait<0>();
  // epilogue: this thread holds rows ((wm*WM + i)*16 + g, + 8) and columns wn*32 + 8j + 2q, +1
#pragma unroll
  for (int i = 0; i < WM; i++)
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int rl = (wm * WM + i) * 16 + g + e * 8;
      if (rl >= rows) continue;
      float wgt = 1.0f;
      size_t orow;
      if (MODE == GM_HEADS) orow = (size_t)group * p.o_hs + (size_t)(row0 + rl) * p.ldo;
      else if (MODE == GM_GATE_UP || MODE == GM_UP) { orow = (size_t)(row0 + rl) * N; wgt = p.wts[src_row[rl]]; }
      else orow = (size_t)src_row[rl] * N;
#pragma unroll
      for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int n = n0 + wn * 32 + 8 * j + 2 * q4 + c;
          if (n >= N) continue;
          const float v = acc[0][i][j][2 * e + c];
          if (MODE == GM_GATE_UP || MODE == GM_UP) {
            const float u = acc[NW - 1][i][j][2 * e + c];
            reinterpret_cast<__nv_bfloat16*>(p.out)[orow + n] =
                __float2bfloat16_rn(moe_pair_act<true>(p.act, p.w_out, p.limit, p.alpha, wgt, v, u));
          } else if (MODE == GM_DOWN || p.out_f32) {
            reinterpret_cast<float*>(p.out)[orow + n] = v;
          } else {
            reinterpret_cast<__nv_bfloat16*>(p.out)[orow + n] = __float2bfloat16_rn(v);
          }
        }
      }
    }
}

template <int MODE, int WM>
static cudaError_t gm_launch(dim3 grid, cudaStream_t stream, const GmArgs& p) {
  static bool set = false;                     // (more than 48 KB of dynamic shared memory must be asked for once)
  if (!set) {
    cudaFuncSetAttribute(grouped_mma_kernel<MODE, WM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GmShape<MODE, WM>::SMEM);
    set = true;
  }
  return tlc_launch(grouped_mma_kernel<MODE, WM>, grid, dim3(128), GmShape<MODE, WM>::SMEM, stream, p);
}

static inline bool gm_aligned(const void* p, long long ld_elems) { return ((uintptr_t)p % 16) == 0 && ld_elems % 8 == 0; }

// Whether the grouped tensor-core product takes these operands: bfloat16, rows that start on 16-byte boundaries.
extern "C" int tlc_grouped_mma_ok(int a_dtype, int w_dtype, const void* a, int lda, int a_hs, const void* w, int K) {
  return a_dtype == TLC_BF16 && w_dtype == TLC_BF16 && K % 8 == 0 && gm_aligned(a, lda) && a_hs % 8 == 0 && gm_aligned(w, K);
}

extern "C" int tlc_linear_heads_mma(const void* a, int lda, int a_hs, const void* w, void* out, int out_dtype, int ldo, int o_hs,
                                    int T, int H, int N, int K, cudaStream_t stream) {
  if (T == 0 || H == 0 || N == 0) return 0;
  TLC_REQUIRE(tlc_grouped_mma_ok(TLC_BF16, TLC_BF16, a, lda, a_hs, w, K), "linear_heads_mma: operands are not aligned for 16-byte copies");
  GmArgs p = {};
  p.a = (const __nv_bfloat16*)a; p.w = (const __nv_bfloat16*)w; p.out = out;
  p.lda = lda; p.a_hs = a_hs; p.ldo = ldo; p.o_hs = o_hs; p.T = T; p.N = N; p.K = K; p.out_f32 = out_dtype == TLC_F32;
  if (T >= 512) {                                           // many rows: 64-row tiles
    gm_launch<GM_HEADS, 2>(dim3((T + 63) / 64, (N + GM_TN - 1) / GM_TN, H), stream, p);
  } else {
    gm_launch<GM_HEADS, 1>(dim3((T + GM_TM - 1) / GM_TM, (N + GM_TN - 1) / GM_TN, H), stream, p);
  }
  TLC_CHECK_LAUNCH("linear_heads_mma");
  return 0;
}

// Both expert products (see moe.cu for the routing arrays): x [T, ldx] bfloat16, wgu [E, 2F, D], wd [E, D, F], act
// [T*top, F] bfloat16 scratch, y [T*top, D] float.
extern "C" int tlc_moe_experts_mma(const void* x, int ldx, const void* wgu, const void* wd, const int* order, const int* offsets,
                                   const int* tile_off, const float* wts, int T, int E, int top, int F, int D, void* act, float* y,
                                   int tile_rows, int act_code, int w_out, float limit, float alpha, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(act_code >= TLC_ACT_SILU && act_code <= TLC_ACT_RELU_SQUARED, "moe_experts_mma: unknown activation %d", act_code);
  TLC_REQUIRE(tile_rows == 32 || tile_rows == 64, "moe_experts_mma: tiles of %d rows are not built (32 or 64, as the routing was made)", tile_rows);
  TLC_REQUIRE(D % 8 == 0 && F % 8 == 0 && gm_aligned(x, ldx) && gm_aligned(wgu, D) && gm_aligned(wd, F) && gm_aligned(act, F),
              "moe_experts_mma: operands are not aligned for 16-byte copies");
  const long long pairs = (long long)T * top;
  const int tiles = (int)(pairs / tile_rows + (pairs < E ? pairs : E));
  GmArgs p = {};
  p.order = order; p.offsets = offsets; p.tile_off = tile_off; p.wts = wts; p.E = E; p.top = top; p.T = T;
  p.act = act_code; p.w_out = w_out; p.limit = limit; p.alpha = alpha;
  p.a = (const __nv_bfloat16*)x; p.lda = ldx; p.w = (const __nv_bfloat16*)wgu; p.out = act; p.N = F; p.K = D;
  if (act_code == TLC_ACT_RELU_SQUARED) {                   // no gate: wgu is [E, F, D], one product
    if (tile_rows == 64) gm_launch<GM_UP, 2>(dim3(tiles, (F + GM_TN - 1) / GM_TN), stream, p);
    else gm_launch<GM_UP, 1>(dim3(tiles, (F + GM_TN - 1) / GM_TN), stream, p);
  } else if (tile_rows == 64) gm_launch<GM_GATE_UP, 2>(dim3(tiles, (F + GM_TN - 1) / GM_TN), stream, p);
  else gm_launch<GM_GATE_UP, 1>(dim3(tiles, (F + GM_TN - 1) / GM_TN), stream, p);
  TLC_CHECK_LAUNCH("moe_gate_up_mma");
  p.a = (const __nv_bfloat16*)act; p.lda = F; p.w = (const __nv_bfloat16*)wd; p.out = y; p.N = D; p.K = F;
  if (tile_rows == 64) gm_launch<GM_DOWN, 2>(dim3(tiles, (D + GM_TN - 1) / GM_TN), stream, p);
  else gm_launch<GM_DOWN, 1>(dim3(tiles, (D + GM_TN - 1) / GM_TN), stream, p);
  TLC_CHECK_LAUNCH("moe_down_mma");
  return 0;
}
