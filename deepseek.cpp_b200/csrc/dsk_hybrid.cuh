// dsk_hybrid.cuh — device kernels of the layer-list ("hybrid") model family: models whose config lists, layer by layer, a
// token mixer (a state-space-duality recurrence or sliding-window latent attention) and an optional routed feed-forward.
// Unlike the persistent batch-1 interpreter (dsk_mega.cuh) these kernels take a CHUNK of T consecutive tokens of one sequence:
// T = 1 is a decode step, T > 1 a prefill portion; the same kernels serve both, reading the recurrent state / latent ring
// cache that the previous chunk left.  Every mechanism is a kernel of its own with its constants as arguments:
//
//   embed_rows        token ids -> fp32 residual rows
//   group_rmsnorm     RMS norm in `groups` equal consecutive parts (groups = 1: plain RMSNorm); can also add its result,
//                     scaled, into the residual, or write its rows into a ring cache
//   gemm_tiled        C = A W^T for T > 4 rows (fp32 activations, fp32 or bf16 weights, fp32 accumulate) with fused
//                     epilogues (residual add, clamped GLU, GELU x per-token embedding) and row gather / scatter / expert tiles
//   gemm_mma          the same interface on the tensor cores for bf16 weights (activations rounded to bf16 as they are staged)
//   gemv_rows         the same interface for T <= 4 rows: one warp per weight row, 16-byte loads
//   causal_conv_silu  depthwise causal convolution over the chunk continuing from the carried (taps - 1) inputs, + SiLU
//   ssd_scan          the state-space recurrence S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, gated by silu(z)
//   latent_swa_attn   softmax attention over a sliding window of cached latents with absorbed key up-projection
//   layer_norm        (x - mean) / sqrt(var + eps) * w, stored or added into the residual
//   qk_norm_rope      RMS norm over a whole query / key projection, partial interleaved rotary positions from a frequency table,
//                     keys and values written into their ring caches
//   gqa_attn          softmax attention of grouped query heads over ring caches of keys and values with a window or chunk mask
//                     and optional mixing of the heads' scores before the softmax (decode-sized steps)
//   pack_ring_kv, mix_heads, softmax_band   the same attention for portions, between three matrix products
//   token_shift       h_t + (h_(t-1) - h_t) * mu in front of a mixer, the last row carried from step to step
//   rms_add_shift_small   decode-sized steps: an RMS-normed addition into the stream and the next layer's token shift in one launch
//   head_rmsnorm      RMS norm per head with one weight vector for all heads
//   hgrn2_scan        the gated linear recurrence S <- diag(f) S + (1 - f) v^T, o = S^T silu(q), f = l + (1 - l) sigmoid(.)
//   moe_route         sigmoid scores, selection by score + correction, weights = normalised scores x scale; or the largest
//                     logits with a softmax over the chosen ones
//   moe_plan          groups the (token, slot) pairs of a chunk by expert into row tiles for gemm_tiled
//   moe_combine       residual += alpha * sum_k w_k y_k (or stored, when a norm follows)
//
// Numerics: the residual stream, norms, router, softmax, recurrent state, decays, step sizes and gates are fp32 in every mode;
// DSK_BF16 models keep their matrices in bfloat16 and accumulate in fp32: decode-sized products multiply them with the fp32
// activations, larger ones round the activations to bfloat16 on their way into the tensor cores.  DSK_F32 models are fp32
// throughout (plain FMA, no reduced-precision matrix mode).
#pragma once

#include <cuda_bf16.h>

#include "dsk_kernels.cuh"

namespace dsk {
namespace hy {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
// log(1 + e^v) without a clamp: beyond 20 the correction term is below half an ulp of v
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__device__ __forceinline__ float block_sum(float v, float* red) {   // red: 33 floats of shared memory; every thread gets the sum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ---------------------------------------------------------------------------------------------------------------------
// conversions at upload: src (fp32 | bf16, row-major rows x cols, pitch src_ld) -> dst (fp32 | bf16).  `tr` > 0 writes the
// per-head transpose of a (heads*tr) x cols matrix: dst[h][c][d] = src[h*tr + d][c] (absorbed key up-projection).
// ---------------------------------------------------------------------------------------------------------------------
template <typename ST, typename DT>
__global__ void convert_kernel(const ST* __restrict__ src, DT* __restrict__ dst, long long rows, long long cols, int tr) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long o = i;
    if (tr > 0) {
      const long long r = i / cols, c = i - r * cols, h = r / tr, d = r - h * tr;
      o = (h * cols + c) * tr + d;
    }
    dst[o] = from_f<DT>(to_f<ST>(src[i]));
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// control words of a chunk: ctl[0] = absolute position of the chunk's first token.  Kept in device memory so that a captured
// decode step can be replayed: advance_ctl moves it on.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void set_ctl(int* ctl, int pos0) { ctl[0] = pos0; }
__global__ void advance_ctl(int* ctl, int by) { ctl[0] += by; }

// x[t] = scale * table[tok[t]] (+ bigram[row]).  The second table is indexed by the pair (previous token, token): row
// (prev * mul_prev + tok * mul_cur) mod buckets, and row `buckets` for the first token of a sequence (position ctl[0] + t == 0).
// The token before the step's first one is carried[0]; carry_token stores the step's last token there afterwards.
template <typename WT>
__global__ void embed_rows(const int* __restrict__ tok, const WT* __restrict__ table, int width, float* __restrict__ x, float scale,
                           const WT* __restrict__ bigram, int buckets, int mul_prev, int mul_cur, const int* __restrict__ ctl,
                           const int* __restrict__ carried) {
  const int t = blockIdx.x;
  const WT* row = table + (size_t)tok[t] * width;
  if (!bigram) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)t * width + c] = scale * to_f<WT>(row[c]);
    return;
  }
  long long r = buckets;
  if (ctl[0] + t > 0) {
    const long long prev = t > 0 ? tok[t - 1] : carried[0];
    r = (prev * mul_prev + (long long)tok[t] * mul_cur) % buckets;
  }
  const WT* brow = bigram + (size_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)t * width + c] = fmaf(scale, to_f<WT>(row[c]), to_f<WT>(brow[c]));
}
// the ring rows of the last taps - 1 positions of a step of T >= taps - 1 tokens (see canon_conv)
__global__ void canon_history(const float* __restrict__ x, int ld, float* __restrict__ hist, int T, int ch, int taps, const int* __restrict__ ctl) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, back = taps - 1;
  if (c >= ch) return;
  for (int j = 0; j < back; j++) {
    const int tau = T - back + j;
    hist[(size_t)((ctl[0] + tau) % back) * ch + c] = x[(size_t)tau * ld + c];
  }
}
__global__ void carry_token(const int* __restrict__ tok, int T, int* __restrict__ carried) { carried[0] = tok[T - 1]; }

// ---------------------------------------------------------------------------------------------------------------------
// Causal per-channel convolution in front of a sublayer, added to its input:  u_t = x_t + sum_j w[c][j] x_(t - taps + 1 + j)
// (the last tap lies on the current token, zeros before the start of the sequence).  `hist` [taps - 1][ch] is a ring over
// positions: the input of position p lives in row p mod (taps - 1).  Thread = channel, CTA = 128 channels x up to 32 consecutive
// tokens; rows of earlier steps come from the ring.  A step of at most 32 tokens (one CTA along the tokens) also stores its
// last taps - 1 inputs in the ring, each thread after its own reads; longer steps run canon_history afterwards, because their
// first CTA reads the rows that the last one would write (taps - 1 <= 16 is required).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kCanonTokens = 32, kCanonMaxTaps = 17;
__global__ void __launch_bounds__(128) canon_conv(const float* __restrict__ x, int ld, const float* __restrict__ w, float* __restrict__ hist,
                                                  float* __restrict__ u, int ldu, int T, int ch, int taps, const int* __restrict__ ctl) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  const int t0 = blockIdx.y * kCanonTokens, t1 = min(T, t0 + kCanonTokens), pos0 = ctl[0], back = taps - 1;
  float wk[kCanonMaxTaps], win[kCanonMaxTaps];   // win[j]: the input `back - j` tokens before the current one
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps; j++) wk[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps - 1; j++) {
    float v = 0.f;
    if (j < back) {
      const int tau = t0 - back + j;          // token index inside the step (negative: an earlier step)
      if (tau >= 0) v = x[(size_t)tau * ld + c];
      else if (pos0 + tau >= 0) v = hist[(size_t)((pos0 + tau) % back) * ch + c];
    }
    win[j] = v;
  }
  for (int t = t0; t < t1; t++) {
    const float cur = x[(size_t)t * ld + c];
    float acc = cur;
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps - 1; j++) if (j < back) acc = fmaf(wk[j], win[j], acc);
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps; j++) if (j == back) acc = fmaf(wk[j], cur, acc);
    u[(size_t)t * ldu + c] = acc;
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps - 2; j++) if (j + 1 < back) win[j] = win[j + 1];
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps - 1; j++) if (j == back - 1) win[j] = cur;
  }
  if (gridDim.y == 1 && back > 0) {   // win now holds the inputs of the last `back` positions (older ones first)
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps - 1; j++) {
      if (j < back) {
        const int p = pos0 + T - back + j;
        if (p >= 0) hist[(size_t)(p % back) * ch + c] = win[j];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// RMS norm in groups.  Row t of `in` (n values) is cut into `groups` equal consecutive parts; each part is divided by
// sqrt(mean(part^2) + eps) and the row is multiplied by w.  mode 0: out[row] = result, where row = (ctl ? ctl[0] : 0) + t,
// taken modulo `ring` (a ring cache of latents; ring = 0 means rows are not wrapped).  mode 1: out[t] += alpha * result.
// ---------------------------------------------------------------------------------------------------------------------
template <typename OT>
__global__ void __launch_bounds__(256) group_rmsnorm(const float* __restrict__ in, int ld_in, const float* __restrict__ w,
                                                     OT* __restrict__ out, int ld_out, int n, int groups, float eps, int mode,
                                                     float alpha, const int* __restrict__ ctl, int ring) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* x = in + (size_t)t * ld_in;
  long long orow = t;
  if (ctl) orow += ctl[0];
  if (ring > 0) orow %= ring;
  OT* o = out + (size_t)orow * ld_out;
  const int gs = n / groups;
  for (int g = 0; g < groups; g++) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = x[g * gs + i]; ss += v * v; }
    ss = block_sum(ss, red);
    const float sc = 1.f / sqrtf(ss / (float)gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
      const int c = g * gs + i;
      const float v = x[c] * sc * w[c];
      if (mode == 0) o[c] = from_f<OT>(v);
      else o[c] = from_f<OT>(to_f<OT>(o[c]) + alpha * v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// matrix products
// ---------------------------------------------------------------------------------------------------------------------
enum { HEPI_STORE = 0, HEPI_ADD = 1, HEPI_GLU = 2, HEPI_GELU_MUL = 3, HEPI_XIELU = 4, HEPI_GEGLU = 5, HEPI_SIGMUL = 6, HEPI_RELU2 = 7, HEPI_LINGATE = 8 };
__host__ __device__ constexpr bool epi_dual(int epi) { return epi == HEPI_GLU || epi == HEPI_GEGLU; }   // two weight matrices per output

struct GemmP {
  const float* A;          // activations, row pitch lda
  const void* W;           // weights [N][K] row-major, row pitch ldw (float or bf16)
  const void* W2;          // HEPI_GLU: the "up" matrix (W is the "gate" matrix)
  float* C;                // row pitch ldc
  int M, N, K, lda, ldw, ldc;
  long long sA, sW, sC;    // element strides per blockIdx.z (per-head batches); sW also is the stride between experts
  int z_wdiv;              // batch z reads weight batch z / z_wdiv (query heads sharing one key / value head)
  const int* a_map;        // logical row i reads A row a_map[i] / a_div (null: row i)
  int a_div;
  const int* c_map;        // logical row i writes C row c_map[i] (null: row i)
  const int* z_expert;     // gemv_rows only: batch z uses expert z_expert[z], A row z / z_adiv, C row z (one row per batch)
  int z_adiv;
  int z_rows;              // gemv_rows only, > 0: batch z takes rows 4z .. 4z + 3 of z_rows rows (narrow outputs over many rows)
  const int4* tiles;       // gemm_tiled only: row tiles grouped by expert {expert, first logical row, rows, -}
  const int* n_tiles;
  float alpha;             // STORE: C = alpha acc; ADD: C += alpha acc
  float lim;               // GLU: g = min(gate, lim), u = clamp(up, -lim, lim), C = g sigmoid(1.702 g) (u + 1)
                           // GEGLU: C = gelu_tanh(gate) * up;  SIGMUL: C *= sigmoid(acc) (a gate on what C already holds);
                           // RELU2: C = max(acc, 0)^2;  LINGATE (the stacked [q | f | v] projection of a gated linear recurrence, aux_off
                           // columns of q and of f): q columns silu(acc), f columns l + (1 - l) sigmoid(acc) with l = aux[n - aux_off] (fp32), v columns acc
  const void* aux;         // GELU_MUL: C = gelu_tanh(acc) * aux[aux_row[row] * aux_ld + aux_off + n]
  const int* aux_row;
  int aux_ld, aux_off;
  const float* bias;       // [N], nullable: added to the accumulator before the epilogue
  float act_a, act_b;      // XIELU: z > 0 ? act_a z^2 + z/2 : act_b (e^z - 1 - z) + z/2
};

template <typename WT, int EPI>
__device__ __forceinline__ void gemm_epilogue(const GemmP& P, float* __restrict__ crow, int cr, int n, float v, float v2) {
  if (P.bias) v += P.bias[n];
  if (EPI == HEPI_STORE) crow[n] = P.alpha * v;
  else if (EPI == HEPI_ADD) crow[n] += P.alpha * v;
  else if (EPI == HEPI_XIELU) crow[n] = v > 0.f ? fmaf(P.act_a * v, v, 0.5f * v) : fmaf(P.act_b, expm1f(v) - v, 0.5f * v);
  else if (EPI == HEPI_GEGLU) crow[n] = gelu_tanh_f(v) * v2;
  else if (EPI == HEPI_SIGMUL) crow[n] *= sigmoid_f(v);
  else if (EPI == HEPI_RELU2) { const float r = fmaxf(v, 0.f); crow[n] = r * r; }
  else if (EPI == HEPI_LINGATE) {
    const int hn = P.aux_off;
    if (n < hn) crow[n] = silu_f(v);
    else if (n < 2 * hn) { const float lo = reinterpret_cast<const float*>(P.aux)[n - hn]; crow[n] = fmaf(1.f - lo, sigmoid_f(v), lo); }
    else crow[n] = v;
  }
  else if (EPI == HEPI_GLU) {
    const float g = fminf(v, P.lim), u = fminf(fmaxf(v2, -P.lim), P.lim);
    crow[n] = g * sigmoid_f(1.702f * g) * (u + 1.f);
  } else {
    const WT* aux = reinterpret_cast<const WT*>(P.aux);
    crow[n] = gelu_tanh_f(v) * to_f<WT>(aux[(size_t)P.aux_row[cr] * P.aux_ld + P.aux_off + n]);
  }
}

// 64 x 64 output tile, K in steps of 16, 256 threads with a 4 x 4 micro-tile each; plain fp32 FMA on fp32 activations.
template <typename WT, int EPI>
__global__ void __launch_bounds__(256) gemm_tiled(const GemmP P) {
  constexpr int BM = 64, BN = 64, BK = 16;
  constexpr bool DUAL = epi_dual(EPI);
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[DUAL ? 2 : 1][BK][BN + 4];
  __shared__ int rowsA[BM], rowsC[BM];
  const int tid = threadIdx.x;
  long long aoff = (long long)blockIdx.z * P.sA, woff = (long long)((int)blockIdx.z / P.z_wdiv) * P.sW, coff = (long long)blockIdx.z * P.sC;
  int row0, nrows;
  if (P.tiles) {
    if ((int)blockIdx.y >= *P.n_tiles) return;
    const int4 t = P.tiles[blockIdx.y];
    woff = (long long)t.x * P.sW;
    row0 = t.y;
    nrows = t.z;
  } else {
    row0 = blockIdx.y * BM;
    nrows = min(BM, P.M - row0);
  }
  if (tid < BM) {
    const int i = row0 + tid;
    const bool ok = tid < nrows;
    rowsA[tid] = ok ? (P.a_map ? P.a_map[i] / P.a_div : i) : -1;
    rowsC[tid] = ok ? (P.c_map ? P.c_map[i] : i) : -1;
  }
  __syncthreads();
  const int n0 = blockIdx.x * BN;
  const WT* __restrict__ W = reinterpret_cast<const WT*>(P.W) + woff;
  const WT* __restrict__ W2 = DUAL ? reinterpret_cast<const WT*>(P.W2) + woff : nullptr;
  const float* __restrict__ A = P.A + aoff;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4], acc2[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) { acc[i][j] = 0.f; acc2[i][j] = 0.f; }
  const int ar = rowsA[lr];
  const int wn = n0 + lr;
  float ra[4], rb[4], rb2[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = k0 + lk + j;
      ra[j] = (ar >= 0 && k < P.K) ? A[(size_t)ar * P.lda + k] : 0.f;
      const bool wok = wn < P.N && k < P.K;
      rb[j] = wok ? to_f<WT>(W[(size_t)wn * P.ldw + k]) : 0.f;
      rb2[j] = (DUAL && wok) ? to_f<WT>(W2[(size_t)wn * P.ldw + k]) : 0.f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < P.K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      As[lk + j][lr] = ra[j];
      Bs[0][lk + j][lr] = rb[j];
      if (DUAL) Bs[DUAL ? 1 : 0][lk + j][lr] = rb2[j];
    }
    __syncthreads();
    if (k0 + BK < P.K) fetch(k0 + BK);   // in flight during this step's FMAs
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[0][kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      if (DUAL) {
        const float4 c4 = *reinterpret_cast<const float4*>(&Bs[DUAL ? 1 : 0][kk][tx * 4]);
        const float c[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int cr = rowsC[ty * 4 + i];
    if (cr < 0) continue;
    float* crow = P.C + coff + (size_t)cr * P.ldc;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < P.N) gemm_epilogue<WT, EPI>(P, crow, cr, n, acc[i][j], acc2[i][j]);
    }
  }
}

// Tensor-core variant for bf16 weights and more than a handful of rows: 128 x 128 tile of A W^T per CTA (K in steps of 32), the
// fp32 activations rounded to bf16 while they are staged, mma.sync m16n8k16 bf16 x bf16 -> fp32.  8 warps as 2 (rows) x 4
// (columns), a 64 x 32 warp tile.  Same row maps, expert tiles, batches and epilogues as gemm_tiled.  For the GLU epilogue the
// 128 staged weight rows alternate, in granules of 8, between the gate and the up matrix, so a thread holds both values of an
// output element in neighbouring accumulators and a CTA produces 64 output columns.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {   // bytes past src_bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kMmaStages = 4;                                   // weight tiles in flight (cp.async ring)
constexpr int kMmaPitch = 40;                                   // bf16 per staged row: 32 + 8 (ldmatrix rows fall on distinct banks)
constexpr size_t kMmaSmem = (size_t)(1 + kMmaStages) * 128 * kMmaPitch * 2;

template <int EPI>
__global__ void __launch_bounds__(256) gemm_mma(const GemmP P) {
  typedef __nv_bfloat16 bf;
  constexpr int BM = 128, BT = 128, BK = 32, PITCH = kMmaPitch, ST = kMmaStages;
  constexpr bool DUAL = epi_dual(EPI);
  constexpr int BN = DUAL ? 64 : 128;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf (*As)[PITCH] = reinterpret_cast<bf (*)[PITCH]>(smraw);                                  // [BM][PITCH]
  bf (*Bs)[BT][PITCH] = reinterpret_cast<bf (*)[BT][PITCH]>(smraw + (size_t)BM * PITCH * 2);   // [ST][BT][PITCH]
  __shared__ int rowsA[BM], rowsC[BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long aoff = (long long)blockIdx.z * P.sA, woff = (long long)((int)blockIdx.z / P.z_wdiv) * P.sW, coff = (long long)blockIdx.z * P.sC;
  int row0, nrows;
  if (P.tiles) {
    if ((int)blockIdx.y >= *P.n_tiles) return;
    const int4 t = P.tiles[blockIdx.y];
    woff = (long long)t.x * P.sW;
    row0 = t.y;
    nrows = t.z;
  } else {
    row0 = blockIdx.y * BM;
    nrows = min(BM, P.M - row0);
  }
  if (tid < BM) {
    const int i = row0 + tid;
    const bool ok = tid < nrows;
    rowsA[tid] = ok ? (P.a_map ? P.a_map[i] / P.a_div : i) : -1;
    rowsC[tid] = ok ? (P.c_map ? P.c_map[i] : i) : -1;
  }
  __syncthreads();
  const int n0 = blockIdx.x * BN;
  const bf* __restrict__ W = reinterpret_cast<const bf*>(P.W) + woff;
  const bf* __restrict__ W2 = DUAL ? reinterpret_cast<const bf*>(P.W2) + woff : nullptr;
  const float* __restrict__ A = P.A + aoff;
  // staging: thread -> (row, 16 consecutive k)
  const int lr = tid >> 1, lk = (tid & 1) * 16;
  const int ar = rowsA[lr];
  int wrow;
  const bf* wsrc = W;
  if (DUAL) { const int g = lr >> 3; wrow = n0 + (g >> 1) * 8 + (lr & 7); wsrc = (g & 1) ? W2 : W; }
  else wrow = n0 + lr;
  const bool wrow_ok = wrow < P.N;
  const bool vecA = (P.lda % 4 == 0) && (aoff % 4 == 0) && (reinterpret_cast<uintptr_t>(P.A) % 16 == 0);
  const bool vecB = (P.ldw % 8 == 0) && (woff % 8 == 0) && (reinterpret_cast<uintptr_t>(P.W) % 16 == 0) &&
                    (!DUAL || reinterpret_cast<uintptr_t>(P.W2) % 16 == 0);
  const int wm = warp & 1, wn = warp >> 1;
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int q = 0; q < 4; q++) acc[i][j][q] = 0.f;
  // The weight stream (from HBM) runs ST - 1 steps ahead through a cp.async ring; the activations (small, L2-resident, fp32 -> bf16
  // on the way) run one step ahead through registers.
  uint32_t ra[8];
  auto fetch_a = [&](int k0) {
    const int kb = k0 + lk;
    if (ar >= 0 && vecA && kb + 16 <= P.K) {
      const float4* src = reinterpret_cast<const float4*>(A + (size_t)ar * P.lda + kb);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float4 v = src[q];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        ra[2 * q] = *reinterpret_cast<const uint32_t*>(&lo);
        ra[2 * q + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const float v0 = (ar >= 0 && kb + 2 * q < P.K) ? A[(size_t)ar * P.lda + kb + 2 * q] : 0.f;
        const float v1 = (ar >= 0 && kb + 2 * q + 1 < P.K) ? A[(size_t)ar * P.lda + kb + 2 * q + 1] : 0.f;
        const __nv_bfloat162 pr = __floats2bfloat162_rn(v0, v1);
        ra[q] = *reinterpret_cast<const uint32_t*>(&pr);
      }
    }
  };
  auto issue_w = [&](int k0, int stage) {   // this thread's 16 weights of K step k0 -> Bs[stage]
    bf* dst = &Bs[stage][lr][lk];
    const int kb = k0 + lk;
    if (vecB) {
      const bool in = wrow_ok && kb < P.K;
      const bf* src = in ? wsrc + (size_t)wrow * P.ldw + kb : wsrc;
      const int left = in ? (P.K - kb) * 2 : 0;                       // valid bytes from kb on
      cp_async_16(dst, src, max(0, min(16, left)));
      cp_async_16(dst + 8, in && left > 16 ? src + 8 : wsrc, max(0, min(16, left - 16)));
    } else {
      const unsigned short* ws = reinterpret_cast<const unsigned short*>(wsrc);
      unsigned short* d = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
      for (int q = 0; q < 16; q++) d[q] = (wrow_ok && kb + q < P.K) ? ws[(size_t)wrow * P.ldw + kb + q] : (unsigned short)0;
    }
  };
  const int nk = (P.K + BK - 1) / BK;
#pragma unroll
  for (int st = 0; st < ST - 1; st++) {
    if (st < nk) issue_w(st * BK, st);
    cp_async_commit();
  }
  fetch_a(0);
  for (int kt = 0; kt < nk; kt++) {
    {
      uint4* da = reinterpret_cast<uint4*>(&As[lr][lk]);
      da[0] = make_uint4(ra[0], ra[1], ra[2], ra[3]); da[1] = make_uint4(ra[4], ra[5], ra[6], ra[7]);
    }
    cp_async_wait<ST - 2>();          // the weights of step kt have landed (one group per step, empty ones included)
    __syncthreads();
    if (kt + ST - 1 < nk) issue_w((kt + ST - 1) * BK, (kt + ST - 1) % ST);   // into the buffer step kt - 1 has finished reading
    cp_async_commit();
    if (kt + 1 < nk) fetch_a((kt + 1) * BK);
    const int sb = kt % ST;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[4][4], bfr[4][2];
      // ldmatrix: lanes 0-7 / 8-15 / 16-23 / 24-31 address the rows of the four 8 x 8 blocks of a fragment
#pragma unroll
      for (int mi = 0; mi < 4; mi++) {
        const int r = wm * 64 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(af[mi], &As[r][kk + (lane >> 4) * 8]);                     // {rows 0-7, k 0-7}, {rows 8-15, k 0-7}, {rows 0-7, k 8-15}, {rows 8-15, k 8-15}
      }
#pragma unroll
      for (int np = 0; np < 2; np++) {
        uint32_t t[4];
        const int n = wn * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(t, &Bs[sb][n][kk + ((lane >> 3) & 1) * 8]);                // {n 0-7, k 0-7}, {n 0-7, k 8-15}, {n 8-15, k 0-7}, {n 8-15, k 8-15}
        bfr[2 * np][0] = t[0]; bfr[2 * np][1] = t[1]; bfr[2 * np + 1][0] = t[2]; bfr[2 * np + 1][1] = t[3];
      }
#pragma unroll
      for (int mi = 0; mi < 4; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++) mma_bf16_16816(acc[mi][ni], af[mi][0], af[mi][1], af[mi][2], af[mi][3], bfr[ni][0], bfr[ni][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int mi = 0; mi < 4; mi++) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int cr = rowsC[wm * 64 + mi * 16 + (lane >> 2) + half * 8];
      if (cr < 0) continue;
      float* crow = P.C + coff + (size_t)cr * P.ldc;
#pragma unroll
      for (int ni = 0; ni < 4; ni += (DUAL ? 2 : 1)) {
#pragma unroll
        for (int q = 0; q < 2; q++) {
          const int g = wn * 4 + ni;   // granule of 8 staged rows
          const int n = DUAL ? n0 + (g >> 1) * 8 + (lane & 3) * 2 + q : n0 + g * 8 + (lane & 3) * 2 + q;
          if (n < P.N) gemm_epilogue<bf, EPI>(P, crow, cr, n, acc[mi][ni][half * 2 + q], DUAL ? acc[mi][ni + 1][half * 2 + q] : 0.f);
        }
      }
    }
  }
}

// Decode-sized steps (T <= kCloseOpenTokens) of post-norm blocks: the end of one sublayer and the start of the next in one kernel,
//   x_t += alpha * rms(y_t) * cw   (cw: norm weight x layer scale);   u_t = x_t + conv(x)_t   with the ring handled as in canon_conv.
// A CTA owns 128 channels over all tokens of the step; every CTA sums the squares of the whole rows of y itself (they are a few
// KB and sit in L2), so no CTA waits for another.
constexpr int kCloseOpenTokens = 8;
__global__ void __launch_bounds__(128) close_open_small(const float* __restrict__ y, const float* __restrict__ cw, float alpha, float eps,
                                                        float* __restrict__ x, int ld, const float* __restrict__ w, float* __restrict__ hist,
                                                        float* __restrict__ u, int T, int ch, int taps, const int* __restrict__ ctl) {
  __shared__ float red[33];
  float sc[kCloseOpenTokens];
#pragma unroll
  for (int t = 0; t < kCloseOpenTokens; t++) {
    if (t < T) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      const float* yr = y + (size_t)t * ld;
      int c = threadIdx.x;
      for (; c + 3 * 128 < ch; c += 4 * 128) {   // four independent loads per round
        const float v0 = yr[c], v1 = yr[c + 128], v2 = yr[c + 256], v3 = yr[c + 384];
        s0 = fmaf(v0, v0, s0); s1 = fmaf(v1, v1, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
      }
      for (; c < ch; c += 128) { const float v = yr[c]; s0 = fmaf(v, v, s0); }
      sc[t] = 1.f / sqrtf(block_sum((s0 + s1) + (s2 + s3), red) / (float)ch + eps);
    } else sc[t] = 0.f;
  }
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= ch) return;
  const int pos0 = ctl[0], back = taps - 1;
  float wk[kCanonMaxTaps], win[kCanonMaxTaps];
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps; j++) wk[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps - 1; j++) {
    const int p = pos0 - back + j;
    win[j] = (j < back && p >= 0) ? hist[(size_t)(p % back) * ch + c] : 0.f;
  }
  const float cwc = cw[c];
#pragma unroll
  for (int t = 0; t < kCloseOpenTokens; t++) {
    if (t < T) {
      const float cur = fmaf(alpha, y[(size_t)t * ld + c] * sc[t] * cwc, x[(size_t)t * ld + c]);
      x[(size_t)t * ld + c] = cur;
      float acc = cur;
#pragma unroll
      for (int j = 0; j < kCanonMaxTaps - 1; j++) if (j < back) acc = fmaf(wk[j], win[j], acc);
#pragma unroll
      for (int j = 0; j < kCanonMaxTaps; j++) if (j == back) acc = fmaf(wk[j], cur, acc);
      u[(size_t)t * ld + c] = acc;
#pragma unroll
      for (int j = 0; j < kCanonMaxTaps - 2; j++) if (j + 1 < back) win[j] = win[j + 1];
#pragma unroll
      for (int j = 0; j < kCanonMaxTaps - 1; j++) if (j == back - 1) win[j] = cur;
    }
  }
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps - 1; j++) {
    if (j < back) {
      const int p = pos0 + T - back + j;
      if (p >= 0) hist[(size_t)(p % back) * ch + c] = win[j];
    }
  }
}

// Decode-sized steps (T <= kCloseOpenTokens): the end of a layer whose last part is an RMS-normed addition, and the token shift that
// opens the next layer, in one kernel:   x_t += alpha * rms(y_t) * w;   hs_t = x_t + (x_(t-1) - x_t) * mu   (mu null: no shift follows).
// `carry` [ch] holds the next layer's input at the token before the step and receives the step's last row.  A CTA owns 128
// channels over all tokens of the step; every CTA sums the squares of the whole rows of y itself, so no CTA waits for another.
__global__ void __launch_bounds__(128) rms_add_shift_small(const float* __restrict__ y, const float* __restrict__ w, float alpha, float eps,
                                                           float* __restrict__ x, int ld, const float* __restrict__ mu, float* __restrict__ carry,
                                                           float* __restrict__ hs, int T, int ch, const int* __restrict__ ctl) {
  __shared__ float red[33];
  float sc[kCloseOpenTokens];
#pragma unroll
  for (int t = 0; t < kCloseOpenTokens; t++) {
    if (t < T) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      const float* yr = y + (size_t)t * ld;
      int c = threadIdx.x;
      for (; c + 3 * 128 < ch; c += 4 * 128) {   // four independent loads per round
        const float v0 = yr[c], v1 = yr[c + 128], v2 = yr[c + 256], v3 = yr[c + 384];
        s0 = fmaf(v0, v0, s0); s1 = fmaf(v1, v1, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
      }
      for (; c < ch; c += 128) { const float v = yr[c]; s0 = fmaf(v, v, s0); }
      sc[t] = 1.f / sqrtf(block_sum((s0 + s1) + (s2 + s3), red) / (float)ch + eps);
    } else sc[t] = 0.f;
  }
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= ch) return;
  const float wc = w[c], m = mu ? mu[c] : 0.f;
  float prev = mu && ctl[0] > 0 ? carry[c] : 0.f;
#pragma unroll
  for (int t = 0; t < kCloseOpenTokens; t++) {
    if (t < T) {
      const float cur = fmaf(alpha, y[(size_t)t * ld + c] * sc[t] * wc, x[(size_t)t * ld + c]);
      x[(size_t)t * ld + c] = cur;
      if (mu) { hs[(size_t)t * ld + c] = fmaf(prev - cur, m, cur); prev = cur; }
    }
  }
  if (mu) carry[c] = prev;
}

template <typename WT> struct WVec;
template <> struct WVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) { const float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <> struct WVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

// M <= 4 rows: one warp per weight row, lanes stride over K with 16-byte loads when pitches and bases allow it.
template <typename WT, int EPI>
__global__ void __launch_bounds__(256) gemv_rows(const GemmP P) {
  constexpr bool DUAL = epi_dual(EPI);
  constexpr int MR = 4, V = WVec<WT>::N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, z = blockIdx.y;
  long long aoff, woff, coff;
  int M = P.M;
  if (P.z_expert) {
    woff = (long long)P.z_expert[z] * P.sW;
    aoff = (long long)(z / P.z_adiv) * P.lda;
    coff = (long long)z * P.ldc;
    M = 1;
  } else if (P.z_rows > 0) {
    aoff = woff = coff = 0;
    M = min(MR, P.z_rows - z * MR);
  } else {
    aoff = (long long)z * P.sA; woff = (long long)(z / P.z_wdiv) * P.sW; coff = (long long)z * P.sC;
  }
  const int mbase = P.z_rows > 0 ? z * MR : 0;
  const WT* __restrict__ W = reinterpret_cast<const WT*>(P.W) + woff;
  const WT* __restrict__ W2 = DUAL ? reinterpret_cast<const WT*>(P.W2) + woff : nullptr;
  const float* arow[MR];
  int crow_i[MR];
#pragma unroll
  for (int m = 0; m < MR; m++) {
    const int mm = mbase + (m < M ? m : 0);
    const int ar = (!P.z_expert && P.a_map) ? P.a_map[mm] / P.a_div : mm;
    arow[m] = P.A + aoff + (size_t)ar * P.lda;
    crow_i[m] = (!P.z_expert && P.c_map) ? P.c_map[mm] : mm;
  }
  const bool vec = (P.K % V == 0) && (P.ldw % V == 0) && (P.lda % 4 == 0) && ((woff * (long long)sizeof(WT)) % 16 == 0) &&
                   ((reinterpret_cast<uintptr_t>(P.W) | (DUAL ? reinterpret_cast<uintptr_t>(P.W2) : 0)) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(P.A + aoff) % 16 == 0);
  for (int n = blockIdx.x * 8 + warp; n < P.N; n += gridDim.x * 8) {
    float acc[MR] = {0.f, 0.f, 0.f, 0.f}, acc2[MR] = {0.f, 0.f, 0.f, 0.f};
    const WT* w = W + (size_t)n * P.ldw;
    const WT* w2 = DUAL ? W2 + (size_t)n * P.ldw : nullptr;
    if (vec) {
#pragma unroll 4
      for (int k = lane * V; k < P.K; k += 32 * V) {   // unrolled: several 16-byte weight loads in flight per lane
        float wv[V], wv2[V];
        WVec<WT>::load(w + k, wv);
        if (DUAL) WVec<WT>::load(w2 + k, wv2);
#pragma unroll
        for (int m = 0; m < MR; m++) {
          if (m < M) {
#pragma unroll
            for (int q = 0; q < V; q += 4) {
              const float4 a = *reinterpret_cast<const float4*>(arow[m] + k + q);
              acc[m] = fmaf(a.x, wv[q], acc[m]); acc[m] = fmaf(a.y, wv[q + 1], acc[m]);
              acc[m] = fmaf(a.z, wv[q + 2], acc[m]); acc[m] = fmaf(a.w, wv[q + 3], acc[m]);
              if (DUAL) {
                acc2[m] = fmaf(a.x, wv2[q], acc2[m]); acc2[m] = fmaf(a.y, wv2[q + 1], acc2[m]);
                acc2[m] = fmaf(a.z, wv2[q + 2], acc2[m]); acc2[m] = fmaf(a.w, wv2[q + 3], acc2[m]);
              }
            }
          }
        }
      }
    } else {
      for (int k = lane; k < P.K; k += 32) {
        const float wv = to_f<WT>(w[k]);
        const float wv2 = DUAL ? to_f<WT>(w2[k]) : 0.f;
#pragma unroll
        for (int m = 0; m < MR; m++) {
          if (m < M) {
            const float a = arow[m][k];
            acc[m] = fmaf(a, wv, acc[m]);
            if (DUAL) acc2[m] = fmaf(a, wv2, acc2[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; m++) {
      if (m < M) {
        const float v = warp_sum(acc[m]);
        const float v2 = DUAL ? warp_sum(acc2[m]) : 0.f;
        if (lane == 0) gemm_epilogue<WT, EPI>(P, P.C + coff + (size_t)crow_i[m] * P.ldc, crow_i[m], n, v, v2);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Depthwise causal convolution + SiLU over a chunk.  in: T rows (pitch ld_in) of `ch` channels; w [ch][taps] with the last tap
// on the current token; `hist` [taps - 1][ch] holds the inputs of the taps - 1 tokens before the chunk (zeros at the start of a
// sequence).  conv_history_update then replaces `hist` with the last taps - 1 inputs seen (it runs after the convolution).
// ---------------------------------------------------------------------------------------------------------------------
__global__ void causal_conv_silu(const float* __restrict__ in, int ld_in, const float* __restrict__ w, const float* __restrict__ b,
                                 const float* __restrict__ hist, float* __restrict__ out, int ld_out, int T, int ch, int taps) {
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  float acc = b[c];
  for (int k = 0; k < taps; k++) {
    const int tau = t - (taps - 1) + k;
    const float v = tau >= 0 ? in[(size_t)tau * ld_in + c] : hist[(size_t)(taps - 1 + tau) * ch + c];
    acc = fmaf(w[(size_t)c * taps + k], v, acc);
  }
  out[(size_t)t * ld_out + c] = silu_f(acc);
}
__global__ void conv_history_update(const float* __restrict__ in, int ld_in, float* __restrict__ hist, int T, int ch, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  for (int j = 0; j < taps - 1; j++) {   // ascending: slot j is read (as slot T + j of the old history) before it is written
    const int tau = T - (taps - 1) + j;
    hist[(size_t)j * ch + c] = tau >= 0 ? in[(size_t)tau * ld_in + c] : hist[(size_t)(taps - 1 + tau) * ch + c];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// State-space-duality recurrence over a chunk, one CTA per (head, slice of PB value channels), sequential over the tokens.
// Thread (pl, s) owns value channel p = p0 + pl and 4 RQ entries of S[h][p][:] (groups of four consecutive n) in registers;
// the eight threads of a channel reduce y with shuffles.  Inputs of TB tokens at a time are staged in shared memory.
//   dt = softplus(raw_dt + dt_bias_h);  S <- exp(-exp(A_log_h) dt) S + dt B x^T;  y = S^T C + D_h x;  out = y silu(z)
// proj: the input projection's rows [z | . | . | . | raw dt]; xbc: the convolved [x | B | C] rows.  Head h reads B/C group h / (H / G).
// ---------------------------------------------------------------------------------------------------------------------
template <int RQ>
__global__ void __launch_bounds__(512) ssd_scan(const float* __restrict__ proj, int ld_proj, int z_off, int dt_off,
                                                const float* __restrict__ xbc, int ld_xbc, int x_off, int b_off, int c_off,
                                                const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                const float* __restrict__ Dskip, float* __restrict__ state,
                                                float* __restrict__ out, int ld_out, int T, int H, int P, int N, int G, int PB, int TB) {
  extern __shared__ __align__(16) float sm[];
  const int NP = (N + 3) & ~3;      // staged B / C rows are padded to whole float4s
  float* s_B = sm;                  // [TB][NP]
  float* s_C = s_B + TB * NP;       // [TB][NP]
  float* s_x = s_C + TB * NP;       // [TB][PB]
  float* s_z = s_x + TB * PB;       // [TB][PB]  silu(z)
  float* s_dt = s_z + TB * PB;      // [TB]
  float* s_dA = s_dt + TB;          // [TB]
  const int h = blockIdx.x, p0 = blockIdx.y * PB, g = h / (H / G);
  const int tid = threadIdx.x, pl = tid >> 3, s = tid & 7, p = p0 + pl;
  const bool pok = pl < PB && p < P;
  // thread (pl, s) owns the state entries n = 4 (s + 8 j) + q, j < RQ, q < 4: one 16-byte shared-memory read per j and operand
  float S[RQ][4];
#pragma unroll
  for (int j = 0; j < RQ; j++)
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int n = 4 * (s + 8 * j) + q;
      S[j][q] = (pok && n < N) ? state[((size_t)h * P + p) * N + n] : 0.f;
    }
  const float a = -expf(A_log[h]), dsk = Dskip[h], dtb = dt_bias[h];
  for (int t0 = 0; t0 < T; t0 += TB) {
    const int nt = min(TB, T - t0);
    __syncthreads();
    for (int i = tid; i < nt; i += blockDim.x) {
      const float dt = softplus_f(proj[(size_t)(t0 + i) * ld_proj + dt_off + h] + dtb);
      s_dt[i] = dt;
      s_dA[i] = expf(a * dt);
    }
    // eight elements per thread and pass: all sixteen loads are in flight before the first is stored (the round is latency-bound)
    for (int base = 0; base < nt * NP; base += 8 * (int)blockDim.x) {
      float vb[8], vc[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * (int)blockDim.x + tid;
        const int tt = i / NP, n = i - tt * NP;
        const bool ok = i < nt * NP && n < N;
        vb[u] = ok ? xbc[(size_t)(t0 + tt) * ld_xbc + b_off + g * N + n] : 0.f;
        vc[u] = ok ? xbc[(size_t)(t0 + tt) * ld_xbc + c_off + g * N + n] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * (int)blockDim.x + tid;
        if (i < nt * NP) { s_B[i] = vb[u]; s_C[i] = vc[u]; }
      }
    }
    for (int base = 0; base < nt * PB; base += 8 * (int)blockDim.x) {
      float vx[8], vz[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * (int)blockDim.x + tid;
        const int tt = i / PB, q = i - tt * PB, pp = p0 + q;
        const bool ok = i < nt * PB && pp < P;
        vx[u] = ok ? xbc[(size_t)(t0 + tt) * ld_xbc + x_off + h * P + pp] : 0.f;
        vz[u] = ok ? proj[(size_t)(t0 + tt) * ld_proj + z_off + h * P + pp] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * (int)blockDim.x + tid;
        if (i < nt * PB) { s_x[i] = vx[u]; s_z[i] = silu_f(vz[u]); }   // the gate, off the sequential path
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; tt++) {
      const float dt = s_dt[tt], dA = s_dA[tt];
      const float xv = pl < PB ? s_x[tt * PB + pl] : 0.f;
      const float dx = dt * xv;
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int j = 0; j < RQ; j++) {
        const int n4 = 4 * (s + 8 * j);
        if (n4 < NP) {   // entries past N are zero in the state and in the staged rows
          const float4 b = *reinterpret_cast<const float4*>(s_B + tt * NP + n4);
          const float4 c = *reinterpret_cast<const float4*>(s_C + tt * NP + n4);
          S[j][0] = fmaf(dA, S[j][0], dx * b.x); S[j][1] = fmaf(dA, S[j][1], dx * b.y);
          S[j][2] = fmaf(dA, S[j][2], dx * b.z); S[j][3] = fmaf(dA, S[j][3], dx * b.w);
          y0 = fmaf(S[j][0], c.x, y0); y1 = fmaf(S[j][1], c.y, y1);
          y0 = fmaf(S[j][2], c.z, y0); y1 = fmaf(S[j][3], c.w, y1);
        }
      }
      float y = y0 + y1;
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 4);
      if (s == 0 && pok) {
        y = fmaf(dsk, xv, y);
        out[(size_t)(t0 + tt) * ld_out + h * P + p] = y * s_z[tt * PB + pl];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < RQ; j++)
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int n = 4 * (s + 8 * j) + q;
      if (pok && n < N) state[((size_t)h * P + p) * N + n] = S[j][q];
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Token shift in front of a mixer:  h_t = x_t + (x_(t-1) - x_t) * mu  per channel, with x_(-1) = 0 at the start of a sequence.
// `carry` [ch] holds the last row of the previous step.  Thread = channel, CTA = 128 channels x up to kCanonTokens consecutive
// tokens.  A step of at most kCanonTokens tokens (one CTA along the tokens) also stores its last row in `carry`, each thread
// after its own read; longer steps run shift_carry afterwards, because their first CTA reads what the last one would write.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) token_shift(const float* __restrict__ x, int ld, const float* __restrict__ mu, float* __restrict__ carry,
                                                   float* __restrict__ h, int ldh, int T, int ch, const int* __restrict__ ctl) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  const int t0 = blockIdx.y * kCanonTokens, t1 = min(T, t0 + kCanonTokens);
  float prev = t0 > 0 ? x[(size_t)(t0 - 1) * ld + c] : (ctl[0] > 0 ? carry[c] : 0.f);
  const float m = mu[c];
  for (int t = t0; t < t1; t++) {
    const float cur = x[(size_t)t * ld + c];
    h[(size_t)t * ldh + c] = fmaf(prev - cur, m, cur);
    prev = cur;
  }
  if (gridDim.y == 1) carry[c] = prev;
}
__global__ void shift_carry(const float* __restrict__ x, int ld, float* __restrict__ carry, int T, int ch) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < ch) carry[c] = x[(size_t)(T - 1) * ld + c];
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated linear recurrence (HGRN2 form) over a chunk, one CTA per (head, slice of PB value channels), sequential over the tokens:
//   S[n][p] <- f[n] S[n][p] + (1 - f[n]) v[p]   (computed as v + f (S - v));   o[p] = sum_n q[n] S[n][p]
// proj rows hold [q | f | v] at the given offsets (H * N, H * N, H * P wide) with the activations already applied by the
// projection's epilogue: q = silu(.), f = l + (1 - l) sigmoid(.) in fp32.  state [H][N][P] fp32.  TPC (8, 16 or 32) threads share a
// value channel: thread (pl, s) owns channel p = p0 + pl and 4 RQ rows n = 4 (s + TPC j) + k of S[:, p] in registers, and the TPC
// threads of a channel reduce o with shuffles.  More threads per channel mean shorter per-token work per thread and more warps to
// hide its latencies (the host picks TPC so that the warps fill the SMs).  Inputs of TB tokens at a time are staged in shared memory.
// ---------------------------------------------------------------------------------------------------------------------
template <int RQ, int TPC>
__global__ void __launch_bounds__(512, 1) hgrn2_scan(const float* __restrict__ proj, int ld, int q_off, int f_off, int v_off,
                                                  float* __restrict__ state, float* __restrict__ out,
                                                  int ld_out, int T, int H, int N, int P, int PB, int TB) {
  extern __shared__ __align__(16) float sm[];
  const int NP = (N + 3) & ~3;      // staged rows are padded to whole float4s
  const int per = TB * (2 * NP + PB);   // floats of one staging buffer: f [TB][NP], q [TB][NP], v [TB][PB]
  const int h = blockIdx.x, p0 = blockIdx.y * PB;
  const int tid = threadIdx.x, pl = tid / TPC, s = tid & (TPC - 1), p = p0 + pl;
  const bool pok = pl < PB && p < P;
  float S[RQ][4];
#pragma unroll
  for (int j = 0; j < RQ; j++)
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int n = 4 * (s + TPC * j) + k;
      S[j][k] = (pok && n < N) ? state[((size_t)h * N + n) * P + p] : 0.f;
    }
  // 16-byte asynchronous copies when every staged run starts on a 16-byte boundary; plain loads otherwise
  const bool vec = (N & 3) == 0 && (ld & 3) == 0 && (q_off & 3) == 0 && (f_off & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
  const bool vecv = vec && (P & 3) == 0 && (PB & 3) == 0 && (v_off & 3) == 0 && p0 + PB <= P;
  // Inputs of TB tokens go into one of two buffers while the recurrence runs over the other
  auto stage = [&](int buf, int t0) {
    float* s_f = sm + buf * per;
    float* s_q = s_f + TB * NP;
    float* s_v = s_q + TB * NP;
    const int nt = min(TB, T - t0);
    if (vec) {
      const int n4 = N >> 2;
      for (int i = tid; i < nt * n4; i += blockDim.x) {
        const int tt = i / n4, c = (i - tt * n4) * 4;
        const float* src = proj + (size_t)(t0 + tt) * ld + h * N + c;
        cp_async_16(s_f + tt * NP + c, src + f_off, 16);
        cp_async_16(s_q + tt * NP + c, src + q_off, 16);
      }
    } else {
      for (int i = tid; i < nt * NP; i += blockDim.x) {
        const int tt = i / NP, n = i - tt * NP;
        const bool ok = n < N;       // padding rows: f = 0, q = 0 (they never reach the output or the stored state)
        s_f[i] = ok ? proj[(size_t)(t0 + tt) * ld + f_off + h * N + n] : 0.f;
        s_q[i] = ok ? proj[(size_t)(t0 + tt) * ld + q_off + h * N + n] : 0.f;
      }
    }
    if (vecv) {
      const int b4 = PB >> 2;
      for (int i = tid; i < nt * b4; i += blockDim.x) {
        const int tt = i / b4, c = (i - tt * b4) * 4;
        cp_async_16(s_v + tt * PB + c, proj + (size_t)(t0 + tt) * ld + v_off + h * P + p0 + c, 16);
      }
    } else {
      for (int i = tid; i < nt * PB; i += blockDim.x) {
        const int tt = i / PB, k = i - tt * PB, pp = p0 + k;
        s_v[i] = pp < P ? proj[(size_t)(t0 + tt) * ld + v_off + h * P + pp] : 0.f;
      }
    }
    cp_async_commit();
  };
  const int nb = (T + TB - 1) / TB;
  stage(0, 0);
  for (int b = 0; b < nb; b++) {
    if (b + 1 < nb) { stage((b + 1) & 1, (b + 1) * TB); cp_async_wait<1>(); }   // the block before the one just issued has landed
    else cp_async_wait<0>();
    __syncthreads();
    const float* s_f = sm + (b & 1) * per;
    const float* s_q = s_f + TB * NP;
    const float* s_v = s_q + TB * NP;
    const int t0 = b * TB, nt = min(TB, T - t0);
#pragma unroll 4
    for (int tt = 0; tt < nt; tt++) {   // unrolled: the loads, the reduction and the shuffles of neighbouring tokens overlap; only S is a chain
      const float xv = pl < PB ? s_v[tt * PB + pl] : 0.f;
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int j = 0; j < RQ; j++) {
        const int n4 = 4 * (s + TPC * j);
        if (n4 < NP) {
          const float4 f = *reinterpret_cast<const float4*>(s_f + tt * NP + n4);
          const float4 c = *reinterpret_cast<const float4*>(s_q + tt * NP + n4);
          S[j][0] = fmaf(f.x, S[j][0] - xv, xv); S[j][1] = fmaf(f.y, S[j][1] - xv, xv);
          S[j][2] = fmaf(f.z, S[j][2] - xv, xv); S[j][3] = fmaf(f.w, S[j][3] - xv, xv);
          y0 = fmaf(S[j][0], c.x, y0); y1 = fmaf(S[j][1], c.y, y1);
          y0 = fmaf(S[j][2], c.z, y0); y1 = fmaf(S[j][3], c.w, y1);
        }
      }
      float y = y0 + y1;
#pragma unroll
      for (int o = 1; o < TPC; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (s == 0 && pok) out[(size_t)(t0 + tt) * ld_out + h * P + p] = y;
    }
    __syncthreads();   // the buffer is free for the block after next
  }
#pragma unroll
  for (int j = 0; j < RQ; j++)
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int n = 4 * (s + TPC * j) + k;
      if (pok && n < N) state[((size_t)h * N + n) * P + p] = S[j][k];
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Sliding-window softmax attention over cached latents with the key up-projection absorbed into the query:
//   score(i, j) = scale * qa[i][h] . c[j]   for  0 <= i - j < window,   o[i][h] = sum_j softmax_j(score) c[j]
// qa [T][H][R] = per-head W_uk^T q; the caller then applies the per-head value up-projection to o [T][H][R].  The latent of
// position j is row j % ring of `cache`.  A CTA of 8 warps takes TQ consecutive tokens x 8 / TQ heads (one warp each) and walks
// the union of their windows in tiles of 32 keys staged in shared memory, so a tile is read once per CTA; lane = key for the
// scores, lane = latent channel (mod 32) for the weighted sum.  Online softmax in fp32.  With NS > 1 (few tokens: decoding) the
// key range is cut into NS shares over blockIdx.z and latent_swa_merge combines the partial results.
// ---------------------------------------------------------------------------------------------------------------------
// first position that position i sees: mask 0 is a sliding window of `size` positions (i included), mask 1 cuts the sequence
// into chunks of `size` positions (borders at multiples of `size`), and i sees its own chunk up to itself
__host__ __device__ __forceinline__ int mask_first(int mask, int size, int i) {
  if (mask == 1) return (i / size) * size;
  return i - size + 1 > 0 ? i - size + 1 : 0;
}

// Row of position j in a cache whose first `keep` rows are fixed (the first positions of a sequence, which a window mask may keep
// visible for ever) and whose other `ring` rows go round:  keep = 0 is a plain ring.
__host__ __device__ __forceinline__ long long cache_row(int j, int keep, int ring) { return j < keep ? j : keep + (j - keep) % ring; }

// What the grouped-query attention kernels do to a scaled score before the softmax, and the softmax's extra denominator term:
//   s <- cap tanh(s / cap) (cap > 0);  s += rel[bucket[min(i - j, rel_max)]][h] (rel non-null; bucket: distance -> row, rel_max + 1 entries);
//   the denominator also holds e^(sink[h]) (sink non-null).  keep: first positions that stay visible under a window mask.
struct ScoreMods {
  float cap;
  const float* rel;
  const int* bucket;
  int rel_max;
  const float* sink;
  int keep;
};
__device__ __forceinline__ float mod_score(const ScoreMods& sm, float s, int dist, int h, int H) {
  if (sm.cap > 0.f) s = sm.cap * tanhf(s / sm.cap);
  if (sm.rel) s += sm.rel[(size_t)sm.bucket[min(dist, sm.rel_max)] * H + h];
  return s;
}

template <typename CT, int RV>
__global__ void __launch_bounds__(256) latent_swa_attn(const float* __restrict__ qa, const CT* __restrict__ cache, float* __restrict__ out,
                                                       int T, int H, int R, const int* __restrict__ ctl, int mask, int window, int ring,
                                                       float scale, int TQ, int NS, float* __restrict__ part) {
  extern __shared__ float sm[];
  const int NW = 8, HB = NW / TQ;
  float* qs = sm;                 // [NW][R]
  float* ks = sm + NW * R;        // [32][R + 1]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int tq0 = blockIdx.x * TQ, t = tq0 + (w % TQ), h = blockIdx.y * HB + w / TQ;
  const bool active = t < T && h < H;
  const int pos0 = ctl[0];
  for (int r = lane; r < R; r += 32) qs[w * R + r] = active ? qa[((size_t)t * H + h) * R + r] * scale : 0.f;
  const int i = pos0 + t;
  const int lo_w = mask_first(mask, window, i), hi_w = i;
  int lo = mask_first(mask, window, pos0 + tq0), hi = pos0 + min(T, tq0 + TQ) - 1;
  if (NS > 1) {   // this CTA's share of the key range (whole tiles of 32)
    const int tiles = (hi - lo + 32) / 32, per = (tiles + NS - 1) / NS;
    const int lo_s = lo + (int)blockIdx.z * per * 32;
    hi = min(hi, lo_s + per * 32 - 1);
    lo = lo_s;
  }
  float m = -1e30f, l = 0.f, acc[RV];
#pragma unroll
  for (int k = 0; k < RV; k++) acc[k] = 0.f;
  for (int j0 = lo; j0 <= hi; j0 += 32) {
    __syncthreads();
    // warp w stages the tile's rows w, w + 8, ..: one ring row index per row, then (fp32 caches of a width that is a multiple of 4)
    // 16-byte loads with all of a lane's loads in flight before the first store
    for (int jj = w; jj < 32; jj += 8) {
      const int j = j0 + jj;
      float* dst = ks + jj * (R + 1);
      if (j > hi) { for (int r = lane; r < R; r += 32) dst[r] = 0.f; continue; }
      const CT* src = cache + (size_t)(j % ring) * R;
      if (sizeof(CT) == 4 && (R & 3) == 0) {
        const float4* s4 = reinterpret_cast<const float4*>(src);
        const int n4 = R >> 2;
#pragma unroll 8
        for (int q = lane; q < n4; q += 32) {
          const float4 v = s4[q];
          dst[4 * q] = v.x; dst[4 * q + 1] = v.y; dst[4 * q + 2] = v.z; dst[4 * q + 3] = v.w;
        }
      } else {
        for (int r = lane; r < R; r += 32) dst[r] = to_f<CT>(src[r]);
      }
    }
    __syncthreads();
    const int j = j0 + lane;
    const bool valid = active && j >= lo_w && j <= hi_w && j <= hi;
    if (!__any_sync(0xffffffffu, valid)) continue;
    const float* kr = ks + lane * (R + 1);
    const float* qr = qs + w * R;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;   // four chains: the dot product is latency-bound otherwise
    int r = 0;
    for (; r + 4 <= R; r += 4) {
      s0 = fmaf(qr[r], kr[r], s0); s1 = fmaf(qr[r + 1], kr[r + 1], s1);
      s2 = fmaf(qr[r + 2], kr[r + 2], s2); s3 = fmaf(qr[r + 3], kr[r + 3], s3);
    }
    for (; r < R; r++) s0 = fmaf(qr[r], kr[r], s0);
    float s = (s0 + s1) + (s2 + s3);
    s = valid ? s : -1e30f;
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int k = 0; k < RV; k++) acc[k] *= corr;
    for (int jj = 0; jj < 32; jj++) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (pj == 0.f) continue;
      const float* c = ks + jj * (R + 1);
#pragma unroll
      for (int k = 0; k < RV; k++) {
        const int r = lane + 32 * k;
        if (r < R) acc[k] = fmaf(pj, c[r], acc[k]);
      }
    }
    m = m_new;
  }
  if (!active) return;
  if (NS > 1) {   // partial result of this key range: [t][h][split] -> {m, l, acc[R]} (not normalised); latent_swa_merge finishes
    float* pp = part + (((size_t)t * H + h) * NS + blockIdx.z) * (R + 2);
    if (lane == 0) { pp[0] = m; pp[1] = l; }
#pragma unroll
    for (int k = 0; k < RV; k++) {
      const int r = lane + 32 * k;
      if (r < R) pp[2 + r] = acc[k];
    }
    return;
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int k = 0; k < RV; k++) {
    const int r = lane + 32 * k;
    if (r < R) out[((size_t)t * H + h) * R + r] = acc[k] * inv;
  }
}

// merges the NS partial softmax results of one (token, head): out = sum_s e^(m_s - m) acc_s / sum_s e^(m_s - m) l_s.
// Grid (token x head, blocks of 128 columns): a thread owns one column and reads its NS partial values with independent loads.
__global__ void __launch_bounds__(128) latent_swa_merge(const float* __restrict__ part, float* __restrict__ out, int R, int NS,
                                                        const float* __restrict__ gate = nullptr, int ld_gate = 0, int H = 1) {
  __shared__ float wts[64], ms[64];   // NS <= 64 (kAttnSplitMax)
  const size_t th = blockIdx.x;
  const float* pp = part + th * NS * (R + 2);
  if ((int)threadIdx.x < NS) ms[threadIdx.x] = pp[(size_t)threadIdx.x * (R + 2)];
  __syncthreads();
  float m = -1e30f;
  for (int s = 0; s < NS; s++) m = fmaxf(m, ms[s]);
  if ((int)threadIdx.x < NS) wts[threadIdx.x] = expf(ms[threadIdx.x] - m);
  __syncthreads();
  float l = 0.f;
  for (int s = 0; s < NS; s++) l = fmaf(wts[s], pp[(size_t)s * (R + 2) + 1], l);
  const float inv = 1.f / l;
  const int r = blockIdx.y * 128 + threadIdx.x;
  if (r >= R) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int s = 0;
  for (; s + 4 <= NS; s += 4) {
    const float v0 = pp[(size_t)s * (R + 2) + 2 + r], v1 = pp[(size_t)(s + 1) * (R + 2) + 2 + r];
    const float v2 = pp[(size_t)(s + 2) * (R + 2) + 2 + r], v3 = pp[(size_t)(s + 3) * (R + 2) + 2 + r];
    a0 = fmaf(wts[s], v0, a0); a1 = fmaf(wts[s + 1], v1, a1); a2 = fmaf(wts[s + 2], v2, a2); a3 = fmaf(wts[s + 3], v3, a3);
  }
  for (; s < NS; s++) a0 = fmaf(wts[s], pp[(size_t)s * (R + 2) + 2 + r], a0);
  // gate (nullable): row th = token * H + head is multiplied by sigmoid(gate[token][head * R + r])
  const float gt = gate ? sigmoid_f(gate[(th / H) * (size_t)ld_gate + (th % H) * (size_t)R + r]) : 1.f;
  out[th * R + r] = ((a0 + a1) + (a2 + a3)) * inv * gt;
}

// out[t][c] *= sigmoid(gate[t][c]) for the n columns of T rows (an output gate whose raw values came out of a stacked projection)
__global__ void gate_rows(float* __restrict__ out, int ld_out, const float* __restrict__ gate, int ld_gate, int n) {
  float* o = out + (size_t)blockIdx.x * ld_out;
  const float* g = gate + (size_t)blockIdx.x * ld_gate;
  for (int c = threadIdx.x; c < n; c += blockDim.x) o[c] *= sigmoid_f(g[c]);
}

// ---------------------------------------------------------------------------------------------------------------------
// Large portions (prefill) run the same attention as three matrix products per block of queries instead: keys and values of the
// visible positions are up-projected from the cached latents (k = W_uk c, v = W_uv c), scores = q k^T per head, a banded softmax,
// then probabilities x values.  The helpers: the ring rows of a run of positions, the per-head repacking of the up-projected
// keys ([head][key][dim]) and values ([head][vdim][key], i.e. transposed, so that both serve as the [N][K] operand of the
// product kernels), and the softmax over the band 0 <= i - j < window of a [head][query][key] score array.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void ring_rows(int first, int n, int ring, int* __restrict__ rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) rows[i] = (first + i) % ring;
}

template <typename WT>
__global__ void pack_keys_values(const float* __restrict__ kf, const float* __restrict__ vf, WT* __restrict__ kb, WT* __restrict__ vt,
                                 int Lk, int H, int D, int V) {
  const int j = blockIdx.x;
  for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
    const int h = e / D, d = e - h * D;
    kb[((size_t)h * Lk + j) * D + d] = from_f<WT>(kf[(size_t)j * H * D + e]);
  }
  for (int e = threadIdx.x; e < H * V; e += blockDim.x) {
    const int h = e / V, v = e - h * V;
    vt[((size_t)h * V + v) * Lk + j] = from_f<WT>(vf[(size_t)j * H * V + e]);
  }
}

// S [H][Tq][Lk] in place: the first nk columns are positions 0 .. nk - 1 (kept first positions that lie before `first`), column
// c >= nk is position first + c - nk; row t is position qpos0 + t and sees j <= i inside its mask or among the kept first
// positions.  Visible scores are modified (ScoreMods) and normalised, hidden entries become 0.
__global__ void __launch_bounds__(128) softmax_band(float* __restrict__ S, int Tq, int Lk, int first, int qpos0, int mask, int window,
                                                    int nk, ScoreMods sm) {
  __shared__ float red[33];
  const int t = blockIdx.x, h = blockIdx.y, H = gridDim.y;
  float* row = S + ((size_t)h * Tq + t) * Lk;
  const int i = qpos0 + t, j_lo = mask_first(mask, window, i);
  float mx = -1e30f;
  for (int c = threadIdx.x; c < Lk; c += blockDim.x) {
    const int j = c < nk ? c : first + c - nk;
    const bool vis = j <= i && (j >= j_lo || j < sm.keep);
    const float v = vis ? mod_score(sm, row[c], i - j, h, H) : -1e30f;
    row[c] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float sink = sm.sink ? sm.sink[h] : -1e30f;
  mx = fmaxf(mx, sink);
  float sum = 0.f;
  for (int c = threadIdx.x; c < Lk; c += blockDim.x) { const float v = row[c]; const float p = v > -1e29f ? expf(v - mx) : 0.f; row[c] = p; sum += p; }
  sum = block_sum(sum, red);
  if (sm.sink) sum += expf(sink - mx);
  const float inv = 1.f / sum;
  for (int c = threadIdx.x; c < Lk; c += blockDim.x) row[c] *= inv;
}

// ---------------------------------------------------------------------------------------------------------------------
// Layer norm with a weight and an optional bias: (x - mean) / sqrt(mean((x - mean)^2) + eps) * w (+ b) per row of n values.
// mode 0: out = result; mode 1: out += alpha * result (a normalised sublayer output added into the residual stream).
// wgt non-null (rows of up to 256 * kLnRegs values): the row that is normalised is the weighted sum of `top` consecutive input
// rows, x_t = sum_k wgt[t * top + k] * in[t * top + k] — the outputs of a token's routed experts, combined on the way in.
// ---------------------------------------------------------------------------------------------------------------------
// A thread keeps its share of the row in registers (rows of up to 256 * kLnRegs values; longer rows are read again).
constexpr int kLnRegs = 16;
__device__ __forceinline__ void ln_stats(const float (&v)[kLnRegs], const float* __restrict__ x, int n, float eps, float* red, float& mean, float& sc) {
  const bool cached = n <= 256 * kLnRegs;
  float s = 0.f;
  if (cached) {
#pragma unroll
    for (int k = 0; k < kLnRegs; k++) s += v[k];        // entries past the row's end are 0
  } else for (int i = threadIdx.x; i < n; i += 256) s += x[i];
  mean = block_sum(s, red) / (float)n;
  float ss = 0.f;
  if (cached) {
#pragma unroll
    for (int k = 0; k < kLnRegs; k++) { const float d = (int)threadIdx.x + 256 * k < n ? v[k] - mean : 0.f; ss = fmaf(d, d, ss); }
  } else for (int i = threadIdx.x; i < n; i += 256) { const float d = x[i] - mean; ss = fmaf(d, d, ss); }
  sc = 1.f / sqrtf(block_sum(ss, red) / (float)n + eps);
}

__global__ void __launch_bounds__(256) layer_norm(const float* __restrict__ in, int ld_in, const float* __restrict__ w, const float* __restrict__ b,
                                                  float* __restrict__ out, int ld_out, int n, float eps, int mode, float alpha,
                                                  const float* __restrict__ wgt, int top) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* x = in + (size_t)t * (wgt ? top : 1) * ld_in;
  float* o = out + (size_t)t * ld_out;
  float v[kLnRegs];
  const bool cached = n <= 256 * kLnRegs;
#pragma unroll
  for (int k = 0; k < kLnRegs; k++) { const int i = threadIdx.x + 256 * k; v[k] = cached && i < n && !wgt ? x[i] : 0.f; }
  if (wgt)
    for (int e = 0; e < top; e++) {
      const float we = wgt[(size_t)t * top + e];
#pragma unroll
      for (int k = 0; k < kLnRegs; k++) { const int i = threadIdx.x + 256 * k; if (i < n) v[k] = fmaf(we, x[(size_t)e * ld_in + i], v[k]); }
    }
  float mean, sc;
  ln_stats(v, x, n, eps, red, mean, sc);
  if (cached) {
#pragma unroll
    for (int k = 0; k < kLnRegs; k++) {
      const int i = threadIdx.x + 256 * k;
      if (i < n) { const float r = (v[k] - mean) * sc * w[i] + (b ? b[i] : 0.f); o[i] = mode == 0 ? r : o[i] + alpha * r; }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += 256) { const float r = (x[i] - mean) * sc * w[i] + (b ? b[i] : 0.f); o[i] = mode == 0 ? r : o[i] + alpha * r; }
  }
}

// The end of one sublayer and the start of the next in one pass over the row (rows of up to 256 * kLnRegs values):
//   x += alpha * ln(y) * wy  (+ row, the vector of a loop pass that opens next);   h = ln(x) * wh
__global__ void __launch_bounds__(256) layer_norm_add_norm(const float* __restrict__ y, const float* __restrict__ wy, float* __restrict__ x,
                                                           const float* __restrict__ row, const float* __restrict__ wh,
                                                           float* __restrict__ h, int n, float eps, float alpha) {
  __shared__ float red[33];
  const size_t t = blockIdx.x;
  const float* yr = y + t * n;
  float* xr = x + t * n;
  float v[kLnRegs];
#pragma unroll
  for (int k = 0; k < kLnRegs; k++) { const int i = threadIdx.x + 256 * k; v[k] = i < n ? yr[i] : 0.f; }
  float mean, sc;
  ln_stats(v, yr, n, eps, red, mean, sc);
#pragma unroll
  for (int k = 0; k < kLnRegs; k++) {
    const int i = threadIdx.x + 256 * k;
    if (i < n) {
      const float r = xr[i] + alpha * ((v[k] - mean) * sc * wy[i]) + (row ? row[i] : 0.f);
      xr[i] = r;
      v[k] = r;
    } else v[k] = 0.f;
  }
  ln_stats(v, xr, n, eps, red, mean, sc);
#pragma unroll
  for (int k = 0; k < kLnRegs; k++) {
    const int i = threadIdx.x + 256 * k;
    if (i < n) h[t * n + i] = (v[k] - mean) * sc * wh[i];
  }
}

// RMS norm of every head of a row with one weight vector shared by the heads: out[t][h][:] = in[t][h][:] / rms(in[t][h][:]) * w[:].
// One warp per (token, head) of P values.
__global__ void __launch_bounds__(256) head_rmsnorm(const float* __restrict__ in, int ld_in, const float* __restrict__ w, float* __restrict__ out,
                                                    int ld_out, int T, int H, int P, float eps) {
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (id >= (long long)T * H) return;
  const int t = (int)(id / H), h = (int)(id - (long long)t * H);
  const float* x = in + (size_t)t * ld_in + (size_t)h * P;
  float* o = out + (size_t)t * ld_out + (size_t)h * P;
  float ss = 0.f;
  for (int i = lane; i < P; i += 32) ss = fmaf(x[i], x[i], ss);
  const float sc = 1.f / sqrtf(warp_sum(ss) / (float)P + eps);
  for (int i = lane; i < P; i += 32) o[i] = x[i] * sc * w[i];
}

// x[t][:] += row[:] for the T rows of a step (the per-pass vector of a layer loop)
__global__ void add_row(float* __restrict__ x, int ld, const float* __restrict__ row, int n) {
  float* o = x + (size_t)blockIdx.x * ld;
  for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] += row[i];
}

// ---------------------------------------------------------------------------------------------------------------------
// Query / key preparation of grouped-query attention, one CTA per token of the step (position ctl[0] + t).
// head_norm == 0:  q <- rot(q / rms(q) * qw),  k <- rot(k / rms(k) * kw)   with the RMS taken over the whole projection (all heads at once);
// head_norm == 1:  q <- rot(q) / rms_head(rot(q)),  k likewise: every head is divided by its own RMS after the rotation, without a weight.
//   rot acts on the first rot_dims dimensions of every head: with layout 0 the pair (2i, 2i + 1) turns by the angle pos * freq[i], with
//   layout 1 the pair (i, i + rot_dims / 2); cos / sin are multiplied by `mag`.  Positions and angles are fp32.
// q (row pitch ld_q; k: ld_k, v_src: ld_v) goes to q_out; the prepared key goes to row cache_row(pos, keep, ring) of kcache.  Values:
// with v_src == nullptr the value of a position is the raw output of its key matrix (ahead of the norm and the rotation);
// otherwise v_src rows are cached, blended with the rows of v_first [T][GV] when that is given: (1 - lam) v + lam v_first.
// v_keep [T][GV], nullable, receives a copy of what is cached (the rows a later layer blends in).
// k == nullptr: a layer that reads another layer's caches prepares its queries only and caches nothing.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float rot_entry(const float* __restrict__ src, int c, int d, int rot_dims, int layout, float nrm, const float* __restrict__ w,
                                           float fpos, const float* __restrict__ freq, float mag) {
  float v = src[c] * nrm * (w ? w[c] : 1.f);
  if (d < rot_dims) {
    const int half = rot_dims >> 1;
    const bool second = layout == 1 ? d >= half : (d & 1);      // which entry of its pair this is
    const int cp = layout == 1 ? (second ? c - half : c + half) : (second ? c - 1 : c + 1);
    const int pi = layout == 1 ? (second ? d - half : d) : (d >> 1);
    const float u = src[cp] * nrm * (w ? w[cp] : 1.f);
    float sn, cs;
    sincosf(fpos * freq[pi], &sn, &cs);
    cs *= mag; sn *= mag;
    v = second ? fmaf(v, cs, u * sn) : fmaf(v, cs, -u * sn);
  }
  return v;
}
__global__ void __launch_bounds__(256) qk_norm_rope(const float* __restrict__ q, float* __restrict__ q_out, int HD,
                                                    const float* __restrict__ k, const float* __restrict__ v_src, int GD, int GV, int ld_q, int ld_k, int ld_v,
                                                    const float* __restrict__ qw, const float* __restrict__ kw, float eps, int D,
                                                    int rot_dims, const float* __restrict__ freq, float mag,
                                                    const int* __restrict__ ctl, float* __restrict__ kcache,
                                                    float* __restrict__ vcache, int ring, int keep, const float* __restrict__ v_first,
                                                    float lam, float* __restrict__ v_keep, int layout, int head_norm) {
  __shared__ float red[33];
  const int t = blockIdx.x, pos = ctl[0] + t;
  const size_t row = (size_t)cache_row(pos, keep, ring);
  const float* qr = q + (size_t)t * ld_q;
  const float* kr = k ? k + (size_t)t * ld_k : nullptr;
  const float fpos = (float)pos;
  if (!k) GD = 0;
  if (head_norm) {   // a warp per head: rotated entries are stored, summed, and scaled by the lane that stored them
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nh = (HD + GD) / D;
    for (int hh = w; hh < nh; hh += 8) {
      const bool isq = hh * D < HD;
      const int c0 = isq ? hh * D : hh * D - HD;
      const float* src = isq ? qr : kr;
      float* dst = isq ? q_out + (size_t)t * HD + c0 : kcache + row * GD + c0;
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float v = rot_entry(src, c0 + d, d, rot_dims, layout, 1.f, nullptr, fpos, freq, mag);
        dst[d] = v;
        ss = fmaf(v, v, ss);
      }
      const float sc = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
      for (int d = lane; d < D; d += 32) dst[d] *= sc;
    }
  } else {
    float sq = 0.f, sk = 0.f;
    for (int e = threadIdx.x; e < HD; e += blockDim.x) sq = fmaf(qr[e], qr[e], sq);
    for (int e = threadIdx.x; e < GD; e += blockDim.x) sk = fmaf(kr[e], kr[e], sk);
    const float nq = qw ? 1.f / sqrtf(block_sum(sq, red) / (float)HD + eps) : 1.f;
    const float nk = kw && k ? 1.f / sqrtf(block_sum(sk, red) / (float)GD + eps) : 1.f;
    for (int e = threadIdx.x; e < HD + GD; e += blockDim.x) {
      const bool isq = e < HD;
      const int c = isq ? e : e - HD, d = c % D;
      const float v = rot_entry(isq ? qr : kr, c, d, rot_dims, layout, isq ? nq : nk, isq ? qw : kw, fpos, freq, mag);
      if (isq) q_out[(size_t)t * HD + c] = v;
      else kcache[row * GD + c] = v;
    }
  }
  if (!k) return;
  const float* vr = v_src ? v_src + (size_t)t * ld_v : kr;
  for (int e = threadIdx.x; e < GV; e += blockDim.x) {
    float v = vr[e];
    if (v_first) v = fmaf(lam, v_first[(size_t)t * GV + e], (1.f - lam) * v);
    vcache[row * GV + e] = v;
    if (v_keep) v_keep[(size_t)t * GV + e] = v;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Grouped-query softmax attention for decode-sized steps: one CTA per (token, share of its keys), all heads in the CTA, because
// the heads' scores may be mixed before the softmax:
//   raw_g(i, j) = scale * q[i][g] . k[j][g / rep];   score_h = sum_g talk[h][g] raw_g   (talk null: score_h = raw_h);
//   o[i][h] = sum_j softmax_j(score_h) v[j][h / rep]   over the positions j that the mask lets i see (mask_first(..) <= j <= i).
// Keys [ring][G*D] and values [ring][G*Dv] are ring caches (position j in row j % ring).  Tiles of 32 keys are staged in shared
// memory; warp w owns heads w, w + 8, ... with their running maximum, sum and weighted value sum in shared memory (online
// softmax, fp32).  NS > 1: the key range is cut into NS shares over blockIdx.y, partial results {m, l, acc[Dv]} go to `part`
// in the layout latent_swa_merge reads.  Without score mixing the key heads may be dealt over gridDim.z CTAs (G / gridDim.z key
// heads with their query heads each), which stage only their own slice of the key rows.  gate (nullable, row pitch ld_gate):
// the output is multiplied by sigmoid(gate[t][h * Dv + r]) (an output gate on the concatenated heads; with NS > 1 the merge does it).
// ---------------------------------------------------------------------------------------------------------------------
__host__ __device__ inline size_t gqa_attn_smem_floats(int H, int G, int D, int Dv) {
  return (size_t)H * D + (size_t)H * 32 + (size_t)32 * (G * D + 1) + 2 * (size_t)H + (size_t)H * Dv + (size_t)H * H + 8 * 32 + 32 + 32;
}
__global__ void __launch_bounds__(256) gqa_attn(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc,
                                                float* __restrict__ out, const float* __restrict__ talk, int T, int H, int G, int D,
                                                int Dv, const int* __restrict__ ctl, int mask, int span, int ring, float scale, int NS,
                                                float* __restrict__ part, ScoreMods mods, const float* __restrict__ gate, int ld_gate) {
  extern __shared__ float sm[];
  const int GD = G * D, GV = G * Dv, rep = H / G;
  const int GL = G / (int)gridDim.z, g0 = (int)blockIdx.z * GL, h0 = g0 * rep, HL = GL * rep, GDl = GL * D;   // this CTA's key heads and query heads
  float* qs = sm;                              // [HL][D]   (the arrays are sized for all heads; a CTA uses the rows of its own)
  float* sc = qs + (size_t)H * D;              // [HL][32] raw scores of the tile
  float* ks = sc + (size_t)H * 32;             // [32][GDl + 1]
  float* ms = ks + (size_t)32 * (GD + 1);      // [HL] running maximum
  float* ls = ms + H;                          // [H] running sum
  float* accs = ls + H;                        // [H][Dv]
  float* tk = accs + (size_t)H * Dv;           // [H][H]
  float* ps = tk + (size_t)H * H;              // [8][32] weights of the warp's current head
  int* rowoff = reinterpret_cast<int*>(ps + 8 * 32);   // [32] cache rows of the tile's keys
  int* kdist = rowoff + 32;                            // [32] their distances from the query
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int t = blockIdx.x, i = ctl[0] + t;
  // the visible keys in one index space: the kept first positions that lie before the mask's range, then the range itself
  const int j_lo = mask_first(mask, span, i), nk = min(mods.keep, j_lo), keep = mods.keep;
  int lo = 0, hi = nk + i - j_lo;
  if (NS > 1) {   // this CTA's share of the keys (whole tiles of 32)
    const int tiles = (hi - lo + 32) / 32, per = (tiles + NS - 1) / NS;
    lo += (int)blockIdx.y * per * 32;
    hi = min(hi, lo + per * 32 - 1);
  }
  auto key_pos = [&](int v) { return v < nk ? v : j_lo + v - nk; };
  for (int e = tid; e < HL * D; e += blockDim.x) qs[e] = q[((size_t)t * H + h0) * D + e];
  for (int e = tid; e < HL; e += blockDim.x) { ms[e] = -1e30f; ls[e] = 0.f; }
  for (int e = tid; e < HL * Dv; e += blockDim.x) accs[e] = 0.f;
  if (talk) for (int e = tid; e < H * H; e += blockDim.x) tk[e] = talk[e];
  for (int j0 = lo; j0 <= hi; j0 += 32) {
    __syncthreads();
    if (tid < 32) {   // keys past the share's end get weight 0 below and any initialised row
      const int p = key_pos(min(j0 + tid, hi));
      rowoff[tid] = (int)cache_row(p, keep, ring);
      kdist[tid] = i - p;
    }
    if ((GD & 3) == 0 && ((D & 3) == 0 || gridDim.z == 1)) {   // 16-byte loads, several in flight per thread (rows and head slices start on 16-byte boundaries)
      const int GD4 = GDl >> 2;
#pragma unroll 8
      for (int e = tid; e < 32 * GD4; e += 256) {
        const int jj = e / GD4, r = (e - jj * GD4) * 4, j = j0 + jj;
        const float4 v = j <= hi ? *reinterpret_cast<const float4*>(kc + (size_t)cache_row(key_pos(j), keep, ring) * GD + g0 * D + r) : make_float4(0.f, 0.f, 0.f, 0.f);
        float* d = ks + jj * (GDl + 1) + r;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
      }
    } else {
      for (int e = tid; e < 32 * GDl; e += blockDim.x) {
        const int jj = e / GDl, r = e - jj * GDl, j = j0 + jj;
        ks[jj * (GDl + 1) + r] = j <= hi ? kc[(size_t)cache_row(key_pos(j), keep, ring) * GD + g0 * D + r] : 0.f;
      }
    }
    __syncthreads();
    for (int hl = w; hl < HL; hl += 8) {   // raw scores: lane = key
      const int h = hl;                  // row of the CTA's own arrays
      const float* kr = ks + lane * (GDl + 1) + (hl / rep) * D;
      const float* qr = qs + h * D;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      int d = 0;
      for (; d + 4 <= D; d += 4) {
        s0 = fmaf(qr[d], kr[d], s0); s1 = fmaf(qr[d + 1], kr[d + 1], s1);
        s2 = fmaf(qr[d + 2], kr[d + 2], s2); s3 = fmaf(qr[d + 3], kr[d + 3], s3);
      }
      for (; d < D; d++) s0 = fmaf(qr[d], kr[d], s0);
      sc[h * 32 + lane] = ((s0 + s1) + (s2 + s3)) * scale;
    }
    __syncthreads();
    const bool valid = j0 + lane <= hi;
    for (int h = w; h < HL; h += 8) {    // h: row of the CTA's own arrays; the head is h0 + h (mixing runs with all heads in one CTA: h0 = 0)
      float s;
      if (talk) {
        s = 0.f;
        for (int g = 0; g < H; g++) s = fmaf(tk[h * H + g], sc[g * 32 + lane], s);
      } else s = sc[h * 32 + lane];
      s = valid ? mod_score(mods, s, kdist[lane], h0 + h, H) : -1e30f;
      const float m_old = ms[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float corr = expf(m_old - m_new);
      const float p = valid ? expf(s - m_new) : 0.f;
      const float l = ls[h] * corr + warp_sum(p);
      ps[w * 32 + lane] = p;
      __syncwarp();
      // weighted values: lane owns columns lane, lane + 32, ... (four at a time); eight keys per batch, so 32 loads are in flight
      // per lane.  Keys past the tile's end have weight 0 and a row inside the ring (initialised memory), so no branch is needed.
      const float* vb = vc + (size_t)((h0 + h) / rep) * Dv;
      const float* pw = ps + w * 32;
      for (int r0 = 0; r0 < Dv; r0 += 128) {
        float a[4];
#pragma unroll
        for (int u = 0; u < 4; u++) { const int r = r0 + lane + 32 * u; a[u] = r < Dv ? accs[h * Dv + r] * corr : 0.f; }
        for (int jj = 0; jj < 32; jj += 8) {
          float v[8][4];
#pragma unroll
          for (int e = 0; e < 8; e++) {
            const float* vr = vb + (size_t)rowoff[jj + e] * GV + r0 + lane;
#pragma unroll
            for (int u = 0; u < 4; u++) v[e][u] = r0 + lane + 32 * u < Dv ? vr[32 * u] : 0.f;
          }
#pragma unroll
          for (int e = 0; e < 8; e++) {
            const float pj = pw[jj + e];
#pragma unroll
            for (int u = 0; u < 4; u++) a[u] = fmaf(pj, v[e][u], a[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) { const int r = r0 + lane + 32 * u; if (r < Dv) accs[h * Dv + r] = a[u]; }
      }
      __syncwarp();
      if (lane == 0) { ms[h] = m_new; ls[h] = l; }
      __syncwarp();
    }
  }
  __syncthreads();
  for (int h = w; h < HL; h += 8) {
    const int hg = h0 + h;                // the head
    float m = ms[h], l = ls[h], corr = 1.f;
    if (mods.sink && blockIdx.y == 0) {   // the sink joins the first share like a key with a zero value vector
      const float sk = mods.sink[hg], m_new = fmaxf(m, sk);
      corr = expf(m - m_new);
      l = l * corr + expf(sk - m_new);
      m = m_new;
    }
    if (NS > 1) {
      float* pp = part + (((size_t)t * H + hg) * NS + blockIdx.y) * (Dv + 2);
      if (lane == 0) { pp[0] = m; pp[1] = l; }
      for (int r = lane; r < Dv; r += 32) pp[2 + r] = accs[h * Dv + r] * corr;
    } else {
      const float inv = corr / l;
      for (int r = lane; r < Dv; r += 32) {
        const float gt = gate ? sigmoid_f(gate[(size_t)t * ld_gate + (size_t)hg * Dv + r]) : 1.f;
        out[((size_t)t * H + hg) * Dv + r] = accs[h * Dv + r] * inv * gt;
      }
    }
  }
}

// Portions run the same attention as matrix products per block of queries (like the latent attention above).  pack_ring_kv
// gathers the visible positions first .. first + Lk - 1 from the ring caches into per-group operands: keys [G][Lk][D], values
// transposed [G][Dv][Lk].  mix_heads applies the heads' score mixing to a [H][Tq][Lk] score array (out of place).
// The first nk operand rows are the kept first positions 0 .. nk - 1 (cache rows of their own, see cache_row).
template <typename WT>
__global__ void pack_ring_kv(const float* __restrict__ kc, const float* __restrict__ vc, WT* __restrict__ kb, WT* __restrict__ vt,
                             int first, int Lk, int ring, int G, int D, int Dv, int nk, int keep) {
  const int j = blockIdx.x;
  const size_t row = (size_t)cache_row(j < nk ? j : first + j - nk, keep, ring);
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int g = e / D, d = e - g * D;
    kb[((size_t)g * Lk + j) * D + d] = from_f<WT>(kc[row * G * D + e]);
  }
  for (int e = threadIdx.x; e < G * Dv; e += blockDim.x) {
    const int g = e / Dv, v = e - g * Dv;
    vt[((size_t)g * Dv + v) * Lk + j] = from_f<WT>(vc[row * G * Dv + e]);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Latent attention with a rotated key part (DSK_MIX_MLA), one CTA per token of the step (position ctl[0] + t):
//   cache row cache_row(pos, 0, ring) <- [ rms(dkv[0:R]) * w  |  rot(dkv[R:R+Rd], pos) ]      (dkv: row pitch ld_dkv)
//   q [T][H][D + Rd]: the last Rd entries of every head are rotated in place;  qa_rot (nullable) [T][H][R + Rd]: the rotated
//   part is also copied behind the R entries that the absorbed key up-projection fills (decode-sized steps score
//   [W_uk^T q_plain | q_rot] against the cache rows directly).
// rot turns the pairs (2i, 2i + 1), i < rot_dims / 2, by pos * freq[i]; positions and angles are fp32.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mla_prepare(const float* __restrict__ dkv, int ld_dkv, const float* __restrict__ w, float eps,
                                                   float* __restrict__ q, float* __restrict__ qa_rot, int H, int D, int Rd, int R,
                                                   int rot_dims, const float* __restrict__ freq, const int* __restrict__ ctl,
                                                   float* __restrict__ cache, int ring) {
  __shared__ float red[33];
  const int t = blockIdx.x, pos = ctl[0] + t, RW = R + Rd;
  const float* src = dkv + (size_t)t * ld_dkv;
  float* crow = cache + (size_t)cache_row(pos, 0, ring) * RW;
  float ss = 0.f;
  for (int e = threadIdx.x; e < R; e += blockDim.x) ss = fmaf(src[e], src[e], ss);
  const float sc = 1.f / sqrtf(block_sum(ss, red) / (float)R + eps);
  for (int e = threadIdx.x; e < R; e += blockDim.x) crow[e] = src[e] * sc * w[e];
  const float fpos = (float)pos;
  const int half = rot_dims >> 1;
  // pairs of the shared key part (head index H) and of every query head
  for (int e = threadIdx.x; e < (H + 1) * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    float sn, cs;
    sincosf(fpos * freq[i], &sn, &cs);
    if (h == H) {
      const float a = src[R + 2 * i], b = src[R + 2 * i + 1];
      crow[R + 2 * i] = a * cs - b * sn;
      crow[R + 2 * i + 1] = b * cs + a * sn;
    } else {
      float* qr = q + ((size_t)t * H + h) * (D + Rd) + D;
      const float a = qr[2 * i], b = qr[2 * i + 1];
      const float ra = a * cs - b * sn, rb = b * cs + a * sn;
      qr[2 * i] = ra; qr[2 * i + 1] = rb;
      if (qa_rot) { float* o = qa_rot + ((size_t)t * H + h) * RW + R; o[2 * i] = ra; o[2 * i + 1] = rb; }
    }
  }
  for (int e = threadIdx.x; e < (H + 1) * (Rd - rot_dims); e += blockDim.x) {   // entries that pass unchanged
    const int h = e / (Rd - rot_dims), d = rot_dims + e - h * (Rd - rot_dims);
    if (h == H) crow[R + d] = src[R + d];
    else if (qa_rot) qa_rot[((size_t)t * H + h) * RW + R + d] = q[((size_t)t * H + h) * (D + Rd) + D + d];
  }
}

// Portions: per-head operands of the score and value products from the up-projected plain keys kf [Lk][H*D], values vf
// [Lk][H*V] and the rotated key parts of the cache rows rows[j] ([R + Rd] each):  kb [H][Lk][D + Rd], vt [H][V][Lk].
__global__ void pack_mla_kv(const float* __restrict__ kf, const float* __restrict__ vf, const float* __restrict__ cache,
                            const int* __restrict__ rows, float* __restrict__ kb, float* __restrict__ vt, int Lk, int H, int D, int Rd,
                            int R, int V) {
  const int j = blockIdx.x, DK = D + Rd;
  const float* kr = cache + (size_t)rows[j] * (R + Rd) + R;
  for (int e = threadIdx.x; e < H * DK; e += blockDim.x) {
    const int h = e / DK, d = e - h * DK;
    kb[((size_t)h * Lk + j) * DK + d] = d < D ? kf[(size_t)j * H * D + h * D + d] : kr[d - D];
  }
  for (int e = threadIdx.x; e < H * V; e += blockDim.x) {
    const int h = e / V, v = e - h * V;
    vt[((size_t)h * V + v) * Lk + j] = vf[(size_t)j * H * V + e];
  }
}

// out[h][e] = sum_g talk[h][g] in[g][e] for the n = Tq * Lk entries of every head; a CTA takes 128 consecutive entries
__global__ void __launch_bounds__(128) mix_heads(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ talk,
                                                 int H, long long n) {
  extern __shared__ float sm[];
  float* tk = sm;              // [H][H]
  float* col = sm + H * H;     // [H][128]
  const long long e = (long long)blockIdx.x * 128 + threadIdx.x;
  for (int k = threadIdx.x; k < H * H; k += blockDim.x) tk[k] = talk[k];
  if (e < n) for (int g = 0; g < H; g++) col[g * 128 + threadIdx.x] = in[(size_t)g * n + e];
  __syncthreads();
  if (e >= n) return;
  for (int h = 0; h < H; h++) {
    float s = 0.f;
    for (int g = 0; g < H; g++) s = fmaf(tk[h * H + g], col[g * 128 + threadIdx.x], s);
    out[(size_t)h * n + e] = s;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Router of a routed feed-forward, one CTA per token.  mode 0: s = sigmoid(logits); the `top` experts with the largest
// s + correction are taken (ties: lower index first), slot = rank; weights = s / (sum of the chosen s + 1e-20) * scale.
// mode 1: the `top` experts with the largest logits are taken (ties: lower index first); weights = softmax over the chosen logits.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void moe_route(const float* __restrict__ logits, const float* __restrict__ correction, int E, int top, float scale,
                          int* __restrict__ idx, float* __restrict__ wgt, int mode) {
  extern __shared__ float sm[];
  float* sc = sm;            // [E]
  float* ch = sm + E;        // [E]
  float* sel = ch + E;       // [top]
  const int t = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float z = logits[(size_t)t * E + e];
    const float s = mode == 1 ? z : sigmoid_f(z);
    sc[e] = s;
    ch[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float c = ch[e];
    int rank = 0;
    for (int i = 0; i < E; i++) rank += (ch[i] > c || (ch[i] == c && i < e)) ? 1 : 0;
    if (rank < top) { idx[(size_t)t * top + rank] = e; sel[rank] = sc[e]; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (mode == 1) {   // slot 0 holds the largest logit
      float sum = 0.f;
      for (int k = 0; k < top; k++) sum += expf(sel[k] - sel[0]);
      for (int k = 0; k < top; k++) wgt[(size_t)t * top + k] = expf(sel[k] - sel[0]) / sum;
    } else {
      float sum = 0.f;
      for (int k = 0; k < top; k++) sum += sel[k];
      const float inv = scale / (sum + 1e-20f);
      for (int k = 0; k < top; k++) wgt[(size_t)t * top + k] = sel[k] * inv;
    }
  }
}

// Groups the `pairs` (token, slot) pairs of a chunk by expert: perm lists the pairs expert by expert (in no particular order
// inside an expert: every row is computed on its own), tiles cuts every expert's run into row tiles of at most `bm` rows
// {expert, first index into perm, rows}.  One CTA: histogram, serial scan over the experts, placement.
__global__ void __launch_bounds__(1024) moe_plan(const int* __restrict__ idx, int pairs, int E, int bm, int* __restrict__ perm,
                                                 int4* __restrict__ tiles, int* __restrict__ n_tiles) {
  extern __shared__ int smi[];
  int* cnt = smi;            // [E]
  int* off = smi + E;        // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < E; e++) {
      off[e] = o;
      for (int r = 0; r < cnt[e]; r += bm) tiles[nt++] = make_int4(e, o + r, min(bm, cnt[e] - r), 0);
      o += cnt[e];
    }
    *n_tiles = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) perm[atomicAdd(&off[idx[i]], 1)] = i;
}

__global__ void moe_combine(float* __restrict__ x, int ldx, const float* __restrict__ y, const float* __restrict__ wgt, int top,
                            int width, float alpha, int add) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; k++) s = fmaf(wgt[(size_t)t * top + k], y[((size_t)t * top + k) * width + c], s);
    x[(size_t)t * ldx + c] = add ? x[(size_t)t * ldx + c] + alpha * s : alpha * s;
  }
}

// arg-max of one logits row -> Ctrl::argmax_key (lowest index on ties), optionally feeding the next token of a device-side
// greedy loop: tok_out[0] = arg-max, log[step] = arg-max.
__global__ void __launch_bounds__(1024) argmax_row(const float* __restrict__ logits, int vocab, Ctrl* __restrict__ ctrl, int* tok_out,
                                                   int* log, int step) {
  __shared__ unsigned long long best[32];
  unsigned long long b = 0ull;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const unsigned long long key = ((unsigned long long)orderable(logits[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
    if (key > b) b = key;
  }
  for (int o = 16; o; o >>= 1) { const unsigned long long v = __shfl_xor_sync(0xffffffffu, b, o); if (v > b) b = v; }
  if ((threadIdx.x & 31) == 0) best[threadIdx.x >> 5] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) if (best[w] > b) b = best[w];
    ctrl->argmax_key = b;
    const int tok = (int)(0xFFFFFFFFu - (unsigned)(b & 0xFFFFFFFFull));
    if (tok_out) tok_out[0] = tok;
    if (log) log[step] = tok;
  }
}

// device-side greedy loop: the token of the last arg-max becomes the next chunk's only token and is logged
__global__ void greedy_feed(const Ctrl* __restrict__ ctrl, int* __restrict__ tok, int* __restrict__ log, int* __restrict__ step) {
  const int t = (int)(0xFFFFFFFFu - (unsigned)(ctrl->argmax_key & 0xFFFFFFFFull));
  tok[0] = t;
  log[*step] = t;
  *step += 1;
}

}  // namespace hy
}  // namespace dsk
