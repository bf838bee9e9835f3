// Kernels of the gated linear recurrent mixer (Griffin's recurrent block with a real-gated linear
// recurrent unit, RG-LRU).  Per channel c of the mixer's width W, for the tokens of one request in
// order:
//
//   u_t   = sum_j conv[c, j] * xin_(t - (taps-1) + j) + conv_b[c]        causal, zeros before the start
//   r_t   = sigmoid(Ra[b] u_t,b + ra_b),  i_t = sigmoid(Ri[b] u_t,b + ri_b)   per block b of W / blocks channels
//   log a = -gain * r_t * softplus(lam[c]),  a_t = exp(log a)
//   S_t   = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t                     S_(-1) = 0
//   out_t = S_t * gelu_tanh(ybranch_t)
//
// xin and ybranch are the two halves of one projection (activation dtype T); everything from u on
// is float: the gates' products are plain FMA chains over the block's channels in index order, so
// a token's gates do not depend on the batch, and the state S is carried in float from step to step.
//
// Per-request state [slots, taps, W] float: row 0 is S, rows 1 .. taps-1 are the last taps-1 inputs
// xin of the request, oldest first (zeros at admission, which are the zeros before the start).
//
// The kernels: the convolution; the two gates of all blocks as one batched FMA product with the
// decay and the input term formed in its epilogue; the scan in chunks over time, which also moves
// the state on.
#include "common.cuh"

#define RG_MAX_TAPS 16

template <typename T>
__global__ void rglru_conv_kernel(const T* __restrict__ yx, int ld, int x_off, const float* __restrict__ conv_w,
                                  const float* __restrict__ conv_b, const float* __restrict__ state,
                                  const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                  const int* __restrict__ slot_ids, float* __restrict__ u, int row0, int width, int taps) {
  pdl_trigger();
  pdl_wait();
  // a row of blocks per token: what depends on the token alone is looked up once
  const int n = row0 + blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int seq = token_seq[n];
  const int first = cu_q[seq];
  const int t = n - first;
  const float* hist = state + ((size_t)slot_ids[seq] * taps + 1) * width + c;      // rows 1 .. taps-1
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int rel = t - (taps - 1) + j;
    const float v = rel >= 0 ? to_f32(yx[(size_t)(first + rel) * ld + x_off + c]) : hist[(size_t)(taps - 1 + rel) * width];
    acc = fmaf(conv_w[(size_t)c * taps + j], v, acc);
  }
  u[(size_t)n * width + c] = acc + conv_b[c];
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// Both gates of every block: for block b (blockIdx.z), rows = tokens, columns = the block's
// channels; two FMA chains per element over the block's input channels in order.  Epilogue:
// a = exp(-gain * sigmoid(ga) * softplus(lam)), bx = sqrt(1 - a^2) * sigmoid(gi) * u.
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
rglru_gates_kernel(const float* __restrict__ u, const float* __restrict__ ra, const float* __restrict__ ra_b,
                   const float* __restrict__ ri, const float* __restrict__ ri_b, const float* __restrict__ lam,
                   float gain, float* __restrict__ a_out, float* __restrict__ bx_out, int n_tokens, int width, int bw) {
  pdl_trigger();
  pdl_wait();
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float Us[BK][BM + 4];
  __shared__ float As[BK][BN + 4];
  __shared__ float Is[BK][BN + 4];
  const int b = blockIdx.z;
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const float* Wa = ra + (size_t)b * bw * bw;
  const float* Wi = ri + (size_t)b * bw * bw;
  float acc_a[TM][TN], acc_i[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc_a[i][j] = acc_i[i][j] = 0.f;
  for (int k0 = 0; k0 < bw; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      Us[c][r] = (gm < n_tokens && gk < bw) ? u[(size_t)gm * width + b * bw + gk] : 0.f;
    }
    for (int e = threadIdx.x; e < BN * BK; e += THREADS) {
      const int r = e / BK, c = e % BK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < bw && gk < bw;
      As[c][r] = ok ? Wa[(size_t)gn * bw + gk] : 0.f;
      Is[c][r] = ok ? Wi[(size_t)gn * bw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float uu[TM], wa[TN], wi[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) uu[i] = Us[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) { wa[j] = As[kk][tx * TN + j]; wi[j] = Is[kk][tx * TN + j]; }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc_a[i][j] = fmaf(uu[i], wa[j], acc_a[i][j]);
          acc_i[i][j] = fmaf(uu[i], wi[j], acc_i[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= bw) continue;
      const int c = b * bw + gn;
      const float r = sigmoid_f(acc_a[i][j] + ra_b[c]);
      const float g = sigmoid_f(acc_i[i][j] + ri_b[c]);
      const float log_a = -gain * r * softplus_f(lam[c]);
      const size_t at = (size_t)gm * width + c;
      a_out[at] = expf(log_a);
      bx_out[at] = sqrtf(-expm1f(2.0f * log_a)) * g * u[at];
    }
  }
}

// The same for steps of few tokens (decode): a CTA takes 16 tokens x 16 channels of one block and
// brings the whole depth of the product into shared memory at once, so that all its loads are in
// flight together instead of a chain of tiles; one thread per (token, channel), the same FMA chains
// in the same order as above.  Dynamic shared memory: 3 x bw x 17 floats.
__global__ void __launch_bounds__(256)
rglru_gates_small_kernel(const float* __restrict__ u, const float* __restrict__ ra, const float* __restrict__ ra_b,
                         const float* __restrict__ ri, const float* __restrict__ ri_b, const float* __restrict__ lam,
                         float gain, float* __restrict__ a_out, float* __restrict__ bx_out, int n_tokens, int width, int bw) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float gates_smem[];
  float* Us = gates_smem;                  // [bw][17]
  float* As = Us + (size_t)bw * 17;
  float* Is = As + (size_t)bw * 17;
  const int b = blockIdx.z, m0 = blockIdx.y * 16, n0 = blockIdx.x * 16;
  const float* Wa = ra + (size_t)b * bw * bw;
  const float* Wi = ri + (size_t)b * bw * bw;
  for (int e = threadIdx.x; e < 16 * bw; e += 256) {
    const int r = e / bw, k = e % bw;                     // consecutive threads read consecutive k
    const int gm = m0 + r, gn = n0 + r;
    Us[k * 17 + r] = gm < n_tokens ? u[(size_t)gm * width + b * bw + k] : 0.f;
    As[k * 17 + r] = gn < bw ? Wa[(size_t)gn * bw + k] : 0.f;
    Is[k * 17 + r] = gn < bw ? Wi[(size_t)gn * bw + k] : 0.f;
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc_a = 0.f, acc_i = 0.f;
  for (int k = 0; k < bw; ++k) {
    const float uu = Us[k * 17 + ty];
    acc_a = fmaf(uu, As[k * 17 + tx], acc_a);
    acc_i = fmaf(uu, Is[k * 17 + tx], acc_i);
  }
  const int gm = m0 + ty, gn = n0 + tx;
  if (gm >= n_tokens || gn >= bw) return;
  const int c = b * bw + gn;
  const float r = sigmoid_f(acc_a + ra_b[c]);
  const float g = sigmoid_f(acc_i + ri_b[c]);
  const float log_a = -gain * r * softplus_f(lam[c]);
  const size_t at = (size_t)gm * width + c;
  a_out[at] = expf(log_a);
  bx_out[at] = sqrtf(-expm1f(2.0f * log_a)) * g * u[at];
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The scan S_t = a_t S_(t-1) + bx_t over an entry's tokens, cut into chunks of RG_CHUNK tokens so
// that long prompts run in parallel over time as well as over channels.
//   rglru_chunk_kernel: one thread per (entry, chunk, channel) folds its chunk into (A, B) with
//     S_end = A S_start + B (A the product of the decays, B the chunk's own sum from zero); the
//     thread of chunk 0 also copies the request's S aside, so that the next kernel never reads the
//     place it writes.
//   rglru_scan_kernel: one thread per (entry, chunk, channel) folds the summaries of the chunks
//     before its own onto the request's S (a short chain of FMAs over values that all chunks of
//     the entry read, so they stay in cache), then runs its chunk and writes out = S * gelu_tanh(y).
//     The thread of the last chunk moves the state on: S, and the last taps-1 inputs of (old
//     inputs ++ this entry's inputs).
// A step whose entries all have up to RG_CHUNK tokens (every decode step) runs the second kernel
// alone: one chunk per entry, S read from the state itself.
// sums: [n_seqs, max_chunks, 2, width] (A, B), then [n_seqs, width] (the requests' S before the step).
#define RG_CHUNK 32

__global__ void rglru_chunk_kernel(const float* __restrict__ a, const float* __restrict__ bx, const float* __restrict__ state,
                                   const int* __restrict__ cu_q, const int* __restrict__ slot_ids, float* __restrict__ sums,
                                   int n_seqs, int width, int taps, int max_chunks) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y, chunk = blockIdx.z;
  const int first = cu_q[seq], n = cu_q[seq + 1] - first;
  if (c >= width || chunk * RG_CHUNK >= n) return;
  if (chunk == 0) sums[(size_t)n_seqs * max_chunks * 2 * width + (size_t)seq * width + c] = state[(size_t)slot_ids[seq] * taps * width + c];
  const int t0 = chunk * RG_CHUNK, t1 = min(n, t0 + RG_CHUNK);
  float A = 1.f, B = 0.f;
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {
    const size_t at = (size_t)(first + t) * width + c;
    const float av = a[at];
    A *= av;
    B = fmaf(av, B, bx[at]);
  }
  const size_t to = ((size_t)seq * max_chunks + chunk) * 2 * width + c;
  sums[to] = A;
  sums[to + width] = B;
}

template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ bx, const T* __restrict__ yx, int ld,
                                  int y_off, int x_off, float* __restrict__ state, const int* __restrict__ cu_q,
                                  const int* __restrict__ slot_ids, T* __restrict__ out, const float* __restrict__ sums,
                                  int n_seqs, int width, int taps, int max_chunks) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y, chunk = blockIdx.z;
  const int first = cu_q[seq], n = cu_q[seq + 1] - first;
  if (c >= width || chunk * RG_CHUNK >= n) return;
  float* st = state + (size_t)slot_ids[seq] * taps * width + c;
  float S = sums ? sums[(size_t)n_seqs * max_chunks * 2 * width + (size_t)seq * width + c] : st[0];
#pragma unroll 8
  for (int j = 0; j < chunk; ++j) {
    const size_t at = ((size_t)seq * max_chunks + j) * 2 * width + c;
    S = fmaf(sums[at], S, sums[at + width]);
  }
  const int t0 = chunk * RG_CHUNK, t1 = min(n, t0 + RG_CHUNK);
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {
    const size_t at = (size_t)(first + t) * width + c;
    S = fmaf(a[at], S, bx[at]);
    out[at] = from_f32<T>(S * gelu_tanh_f(to_f32(yx[(size_t)(first + t) * ld + y_off + c])));
  }
  if (t1 < n) return;                          // the last chunk's thread moves the state on; nobody else reads it here
  st[0] = S;
  float keep[RG_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < RG_MAX_TAPS - 1; ++k) {
    if (k < taps - 1) {
      const int rel = n - (taps - 1) + k;
      keep[k] = rel >= 0 ? to_f32(yx[(size_t)(first + rel) * ld + x_off + c]) : st[(size_t)(1 + k + n) * width];
    }
  }
#pragma unroll
  for (int k = 0; k < RG_MAX_TAPS - 1; ++k)
    if (k < taps - 1) st[(size_t)(1 + k) * width] = keep[k];
}

template <typename T>
static int rglru_conv(const void* yx, int ld, int x_off, const float* conv_w, const float* conv_b, const float* state,
                      const int* token_seq, const int* cu_q, const int* slot_ids, float* u, int n_tokens, int width, int taps,
                      void* stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > RG_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (n_tokens > 65535 * 32) return (int)cudaErrorInvalidValue;
  for (int at = 0; at < n_tokens; at += 65535) {                  // the grid's second dimension ends at 65,535
    const int rows = n_tokens - at < 65535 ? n_tokens - at : 65535;
    launch(rglru_conv_kernel<T>, dim3((width + 255) / 256, rows), dim3(256), 0, (cudaStream_t)stream, (const T*)yx, ld, x_off, conv_w,
           conv_b, state, token_seq, cu_q, slot_ids, u, at, width, taps);
  }
  return launch_status();
}

// Floats of scratch memory the scan needs for a step whose longest entry has max_q_len tokens (0: none).
Q25_EXPORT long long q25_rglru_scan_scratch_floats(int n_seqs, int max_q_len, int width) {
  const int max_chunks = (max_q_len + RG_CHUNK - 1) / RG_CHUNK;
  return max_chunks <= 1 ? 0 : (long long)n_seqs * width * (2 * max_chunks + 1);
}

template <typename T>
static int rglru_scan(const float* a, const float* bx, const void* yx, int ld, int y_off, int x_off, float* state, const int* cu_q,
                      const int* slot_ids, void* out, int n_seqs, int max_q_len, float* sums, int width, int taps, void* stream) {
  if (n_seqs <= 0) return 0;
  if (taps < 1 || taps > RG_MAX_TAPS || max_q_len < 1) return (int)cudaErrorInvalidValue;
  const int max_chunks = (max_q_len + RG_CHUNK - 1) / RG_CHUNK;
  if (max_chunks > 65535 || (max_chunks > 1 && !sums)) return (int)cudaErrorInvalidValue;
  const dim3 grid((width + 127) / 128, n_seqs, max_chunks);
  if (max_chunks > 1)
    launch(rglru_chunk_kernel, grid, dim3(128), 0, (cudaStream_t)stream, a, bx, (const float*)state, cu_q, slot_ids, sums, n_seqs, width,
           taps, max_chunks);
  launch(rglru_scan_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, a, bx, (const T*)yx, ld, y_off, x_off, state, cu_q, slot_ids,
         (T*)out, (const float*)(max_chunks > 1 ? sums : nullptr), n_seqs, width, taps, max_chunks);
  return launch_status();
}

Q25_EXPORT int q25_rglru_conv_f32(const void* yx, int ld, int xo, const float* cw, const float* cb, const float* st, const int* ts,
                                  const int* cu, const int* sl, float* u, int n, int w, int taps, void* s) {
  return rglru_conv<float>(yx, ld, xo, cw, cb, st, ts, cu, sl, u, n, w, taps, s);
}
Q25_EXPORT int q25_rglru_conv_bf16(const void* yx, int ld, int xo, const float* cw, const float* cb, const float* st, const int* ts,
                                   const int* cu, const int* sl, float* u, int n, int w, int taps, void* s) {
  return rglru_conv<bf16>(yx, ld, xo, cw, cb, st, ts, cu, sl, u, n, w, taps, s);
}
Q25_EXPORT int q25_rglru_gates(const float* u, const float* ra, const float* ra_b, const float* ri, const float* ri_b,
                               const float* lam, float gain, float* a_out, float* bx_out, int n_tokens, int width, int blocks,
                               void* stream) {
  if (n_tokens <= 0) return 0;
  if (blocks <= 0 || width % blocks) return (int)cudaErrorInvalidValue;
  const int bw = width / blocks;
  const size_t small_smem = (size_t)3 * bw * 17 * sizeof(float);
  if (n_tokens <= 128 && small_smem <= 160 * 1024) {
    if (small_smem > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(rglru_gates_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)small_smem);
      if (e != cudaSuccess) return (int)e;
    }
    launch(rglru_gates_small_kernel, dim3((bw + 15) / 16, (n_tokens + 15) / 16, blocks), dim3(256), small_smem, (cudaStream_t)stream, u, ra,
           ra_b, ri, ri_b, lam, gain, a_out, bx_out, n_tokens, width, bw);
  } else if (n_tokens <= 16) {
    launch(rglru_gates_kernel<16, 64, 16, 1, 4>, dim3((bw + 63) / 64, (n_tokens + 15) / 16, blocks), dim3(256), 0, (cudaStream_t)stream,
           u, ra, ra_b, ri, ri_b, lam, gain, a_out, bx_out, n_tokens, width, bw);
  } else {
    launch(rglru_gates_kernel<64, 64, 16, 4, 4>, dim3((bw + 63) / 64, (n_tokens + 63) / 64, blocks), dim3(256), 0, (cudaStream_t)stream,
           u, ra, ra_b, ri, ri_b, lam, gain, a_out, bx_out, n_tokens, width, bw);
  }
  return launch_status();
}
Q25_EXPORT int q25_rglru_scan_f32(const float* a, const float* bx, const void* yx, int ld, int yo, int xo, float* st, const int* cu,
                                  const int* sl, void* out, int n_seqs, int max_q_len, float* sums, int w, int taps, void* s) {
  return rglru_scan<float>(a, bx, yx, ld, yo, xo, st, cu, sl, out, n_seqs, max_q_len, sums, w, taps, s);
}
Q25_EXPORT int q25_rglru_scan_bf16(const float* a, const float* bx, const void* yx, int ld, int yo, int xo, float* st, const int* cu,
                                   const int* sl, void* out, int n_seqs, int max_q_len, float* sums, int w, int taps, void* s) {
  return rglru_scan<bf16>(a, bx, yx, ld, yo, xo, st, cu, sl, out, n_seqs, max_q_len, sums, w, taps, s);
}
