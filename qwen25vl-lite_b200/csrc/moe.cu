// Kernels of the routed feed-forward (a mixture of small gated feed-forwards, of which each token
// uses `top`):
//
//   z = Wr h (float), s = sigmoid(z); the `top` experts with the largest scores, weights s (as they are)
//   expert e on input a = s_e * h:  g = min(Wg a, limit), u = clamp(Wu a, -limit, limit),
//                                   y = Wd (g * sigmoid(alpha g) * (u + 1))
//   out = sum over the chosen experts of y  (+ sigmoid(Wsg h) * shared(h), the caller's product)
//
// The (token, expert) pairs of a step are sorted by expert on the device: the router counts, a
// one-block kernel lays the experts' rows out one after the other (each expert's rows filled up to
// a whole number of row tiles), a scatter kernel gives every pair its row.  Two grouped products
// then walk the row tiles, each tile belonging to one expert: gate and up with the activation in
// the epilogue, and down.  A last kernel adds a token's rows up in the order of its choices.
// Nothing is read back by the host, so a step can be captured into a graph; the grids are sized
// for the most tiles there can be and the tiles past the count leave at once.
//
// Every output element of the plain products is one FMA chain over k in order, whatever tile the
// row falls into, so a token's result does not depend on the batch.  The bfloat16 products run on
// the tensor cores (mma.sync m16n8k16, float accumulators) with the same layout.
#include "attention_decode.cuh"

#define MOE_MAX_EXPERTS 256
#define MOE_MAX_TOP 16

// One warp per token: router logits in float (the lanes stride over the channels, then a butterfly:
// a fixed order), the choice of the `top` largest (ties to the lower index), the shared expert's gate.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ shared_gate,
                                 int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ sg,
                                 int* __restrict__ counts, int n_tokens, int hidden, int experts, int top) {
  pdl_trigger();
  pdl_wait();
  __shared__ float zs[4][MOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  if (n >= n_tokens) return;
  const T* row = h + (size_t)n * hidden;
  for (int e = 0; e < experts; ++e) {
    const float* w = router + (size_t)e * hidden;
    float acc = 0.f;
    for (int c = lane; c < hidden; c += 32) acc = fmaf(w[c], to_f32(row[c]), acc);
    acc = warp_sum(acc);
    if (lane == 0) zs[warp][e] = acc;
  }
  if (shared_gate) {
    float acc = 0.f;
    for (int c = lane; c < hidden; c += 32) acc = fmaf(shared_gate[c], to_f32(row[c]), acc);
    acc = warp_sum(acc);
    if (lane == 0) sg[n] = 1.0f / (1.0f + expf(-acc));
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float z = zs[warp][e];
      if (z > best) { best = z; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) {
      topk_idx[(size_t)n * top + k] = arg;
      topk_w[(size_t)n * top + k] = 1.0f / (1.0f + expf(-best));
      zs[warp][arg] = -INFINITY;
      atomicAdd(&counts[arg], 1);
    }
    __syncwarp();
  }
}

// One block: where every expert's rows begin (each expert filled up to whole tiles of `tile` rows),
// which expert every tile belongs to, how many tiles there are; all rows marked empty.
// plan: [0] number of tiles, [1 .. experts+1] first row of each expert (and the end), then the tiles' experts.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ plan, int* __restrict__ row_pair,
                                int experts, int tile, int max_rows) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    int row = 0, t = 0;
    int* first = plan + 1;
    int* tile_expert = plan + 2 + experts;
    for (int e = 0; e < experts; ++e) {
      first[e] = row;
      const int tiles = (counts[e] + tile - 1) / tile;
      for (int i = 0; i < tiles; ++i) tile_expert[t++] = e;
      row += tiles * tile;
    }
    first[experts] = row;
    plan[0] = t;
  }
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_pair[r] = -1;
}

__global__ void moe_scatter_kernel(const int* __restrict__ topk_idx, const int* __restrict__ plan, int* __restrict__ cursor,
                                   int* __restrict__ row_pair, int* __restrict__ pair_row, int n_pairs) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * blockDim.x + threadIdx.x;
  if (pair >= n_pairs) return;
  const int e = topk_idx[pair];
  const int r = plan[1 + e] + atomicAdd(&cursor[e], 1);
  row_pair[r] = pair;
  pair_row[pair] = r;
}

// Grouped product on the CUDA cores.  GATE_UP: rows are the tile's pairs, a = weight * h[token];
// two chains per element (gate, up), activation in the epilogue, out = act [rows, N] in T.
// Otherwise: rows are act rows, one chain, out = y [rows, N] in float.  W* are [experts, N, K].
template <typename T, bool GATE_UP, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
moe_grouped_fma_kernel(const T* __restrict__ A, const T* __restrict__ W0, const T* __restrict__ W1, void* __restrict__ out_,
                       const int* __restrict__ plan, const int* __restrict__ row_pair, const float* __restrict__ topk_w,
                       int experts, int top, int N, int K, float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  constexpr int THREADS = (BM / TM) * (BN / TN);
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[2 + experts + tile];
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws0[BK][BN + 4];
  __shared__ float Ws1[GATE_UP ? BK : 1][BN + 4];
  __shared__ int src_row[BM];
  __shared__ float src_w[BM];
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = threadIdx.x; r < BM; r += THREADS) {
    const int pair = row_pair[m0 + r];
    if (GATE_UP) {
      src_row[r] = pair < 0 ? -1 : pair / top;
      src_w[r] = pair < 0 ? 0.f : topk_w[pair];
    } else {
      src_row[r] = pair < 0 ? -1 : m0 + r;
      src_w[r] = 1.f;
    }
  }
  __syncthreads();
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const T* w0 = W0 + (size_t)e * N * K;
  const T* w1 = GATE_UP ? W1 + (size_t)e * N * K : nullptr;
  float acc0[TM][TN], acc1[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc0[i][j] = acc1[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int x = threadIdx.x; x < BM * BK; x += THREADS) {
      const int r = x / BK, c = x % BK;
      const int gk = k0 + c, src = src_row[r];
      float v = 0.f;
      if (src >= 0 && gk < K) v = to_f32(A[(size_t)src * K + gk]);
      As[c][r] = GATE_UP ? v * src_w[r] : v;
    }
    for (int x = threadIdx.x; x < BN * BK; x += THREADS) {
      const int r = x / BK, c = x % BK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < N && gk < K;
      Ws0[c][r] = ok ? to_f32(w0[(size_t)gn * K + gk]) : 0.f;
      if (GATE_UP) Ws1[c][r] = ok ? to_f32(w1[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b0[TN], b1[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b0[j] = Ws0[kk][tx * TN + j];
        if (GATE_UP) b1[j] = Ws1[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc0[i][j] = fmaf(a[i], b0[j], acc0[i][j]);
          if (GATE_UP) acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (src_row[r] < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (GATE_UP) {
        const float g = fminf(acc0[i][j], limit);
        const float u = fminf(fmaxf(acc1[i][j], -limit), limit);
        reinterpret_cast<T*>(out_)[(size_t)(m0 + r) * N + gn] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
      } else {
        reinterpret_cast<float*>(out_)[(size_t)(m0 + r) * N + gn] = acc0[i][j];
      }
    }
  }
}

// The grouped products on the tensor cores (bfloat16, mma.sync m16n8k16, float accumulators): a CTA
// of 4 warps takes a tile of BM rows x 64 columns of one expert; with BM = 64 a warp holds 16 rows and
// all 64 columns, with BM = 16 all rows and 16 columns.  K is walked in steps of 32: the weights'
// rows by 16-byte cp.async, the rows of A by plain loads (gate and up: the token's row times its
// weight, rounded to bfloat16), one stage: several CTAs share an SM and hide each other's loads.
// Every element's sum runs over K in the same order whatever tile the row is in.
template <bool GATE_UP, int BM>
__global__ void __launch_bounds__(128)
moe_grouped_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W0, const bf16* __restrict__ W1, void* __restrict__ out_,
                       const int* __restrict__ plan, const int* __restrict__ row_pair, const float* __restrict__ topk_w,
                       int experts, int top, int N, int K, float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  constexpr int BN = 64, BK = 32, P = BK * 2 + 16;            // pitch in bytes: an odd number of 16-byte chunks
  constexpr int WN = BM == 64 ? 64 : 16;                      // columns a warp holds
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[2 + experts + tile];
  __shared__ __align__(16) unsigned char As[BM * P];
  __shared__ __align__(16) unsigned char Ws0[BN * P];
  __shared__ __align__(16) unsigned char Ws1[GATE_UP ? BN * P : 16];
  __shared__ int src_row[BM];
  __shared__ float src_w[BM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = threadIdx.x; r < BM; r += 128) {
    const int pair = row_pair[m0 + r];
    src_row[r] = pair < 0 ? -1 : (GATE_UP ? pair / top : m0 + r);
    src_w[r] = (GATE_UP && pair >= 0) ? topk_w[pair] : 1.f;
  }
  __syncthreads();
  const bf16* w0 = W0 + (size_t)e * N * K;
  const bf16* w1 = GATE_UP ? W1 + (size_t)e * N * K : nullptr;
  const int row_base = BM == 64 ? warp * 16 : 0, col_base = BM == 64 ? 0 : warp * 16;
  float acc0[WN / 8][4], acc1[GATE_UP ? WN / 8 : 1][4];
#pragma unroll
  for (int j = 0; j < WN / 8; ++j) acc0[j][0] = acc0[j][1] = acc0[j][2] = acc0[j][3] = 0.f;
  if (GATE_UP) {
#pragma unroll
    for (int j = 0; j < WN / 8; ++j) acc1[j][0] = acc1[j][1] = acc1[j][2] = acc1[j][3] = 0.f;
  }
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int x = threadIdx.x; x < BN * (BK / 8); x += 128) {
      const int r = x / (BK / 8), ch = x % (BK / 8);
      const int gn = n0 + r, gk = k0 + ch * 8;
      const bool ok = gn < N && gk < K;
      const size_t off = ok ? (size_t)gn * K + gk : 0;
      cp_async16(Ws0 + r * P + ch * 16, w0 + off, ok);
      if (GATE_UP) cp_async16(Ws1 + r * P + ch * 16, w1 + off, ok);
    }
    cp_async_commit();
    for (int x = threadIdx.x; x < BM * (BK / 8); x += 128) {
      const int r = x / (BK / 8), ch = x % (BK / 8);
      const int gk = k0 + ch * 8, src = src_row[r];
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (src >= 0 && gk < K) {
        v = *reinterpret_cast<const uint4*>(A + (size_t)src * K + gk);
        if (GATE_UP) {
          const float w = src_w[r];
          unsigned* u = reinterpret_cast<unsigned*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u[i]);
            u[i] = pack_bf16(__low2float(b) * w, __high2float(b) * w);
          }
        }
      }
      *reinterpret_cast<uint4*>(As + r * P + ch * 16) = v;
    }
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      unsigned a[4];
      ldmatrix_x4(a, As + (row_base + (lane & 15)) * P + (kk * 16 + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int j = 0; j < WN / 8; ++j) {
        unsigned b[2];
        ldmatrix_x2(b, Ws0 + (col_base + j * 8 + (lane & 7)) * P + (kk * 16 + 8 * ((lane >> 3) & 1)) * 2);
        mma_bf16(acc0[j], a, b[0], b[1]);
        if (GATE_UP) {
          ldmatrix_x2(b, Ws1 + (col_base + j * 8 + (lane & 7)) * P + (kk * 16 + 8 * ((lane >> 3) & 1)) * 2);
          mma_bf16(acc1[j], a, b[0], b[1]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < WN / 8; ++j) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = row_base + g + 8 * half;
      if (src_row[r] < 0) continue;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int gn = n0 + col_base + j * 8 + 2 * t + c;
        if (gn >= N) continue;
        const float v0 = acc0[j][2 * half + c];
        if (GATE_UP) {
          const float gt = fminf(v0, limit);
          const float up = fminf(fmaxf(acc1[j][2 * half + c], -limit), limit);
          reinterpret_cast<bf16*>(out_)[(size_t)(m0 + r) * N + gn] = __float2bfloat16_rn(gt / (1.0f + expf(-alpha * gt)) * (up + 1.0f));
        } else {
          reinterpret_cast<float*>(out_)[(size_t)(m0 + r) * N + gn] = v0;
        }
      }
    }
  }
}

// out[n, :] = sum over the token's choices, in their order, of y[row of the pair, :]
//             (+ sg[n] * shared[n, :]), in T.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ sg,
                                   const T* __restrict__ shared, T* __restrict__ out, int n_tokens, int hidden, int top) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_tokens * hidden;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(i / hidden), c = (int)(i % hidden);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc += y[(size_t)pair_row[(size_t)n * top + k] * hidden + c];
    if (shared) acc = fmaf(sg[n], to_f32(shared[i]), acc);
    out[i] = from_f32<T>(acc);
  }
}

// Rows that the sorted pairs can take at most: every pair, and each expert filled up to a tile.
Q25_EXPORT int q25_moe_max_rows(int n_pairs, int experts, int tile) {
  const int most_tiles = (n_pairs + tile - 1) / tile + experts;
  return most_tiles * tile;
}

template <typename T>
static int moe_route(const void* h, const float* router, const float* shared_gate, int* topk_idx, float* topk_w, float* sg,
                     int* counts, int n_tokens, int hidden, int experts, int top, void* stream) {
  if (n_tokens <= 0) return 0;
  if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || top > MOE_MAX_TOP) return (int)cudaErrorInvalidValue;
  launch(moe_route_kernel<T>, dim3((n_tokens + 3) / 4), dim3(128), 0, (cudaStream_t)stream, (const T*)h, router, shared_gate, topk_idx,
         topk_w, sg, counts, n_tokens, hidden, experts, top);
  return launch_status();
}

Q25_EXPORT int q25_moe_route_f32(const void* h, const float* r, const float* g, int* ti, float* tw, float* sg, int* counts, int n,
                                 int hidden, int experts, int top, void* s) {
  return moe_route<float>(h, r, g, ti, tw, sg, counts, n, hidden, experts, top, s);
}
Q25_EXPORT int q25_moe_route_bf16(const void* h, const float* r, const float* g, int* ti, float* tw, float* sg, int* counts, int n,
                                  int hidden, int experts, int top, void* s) {
  return moe_route<bf16>(h, r, g, ti, tw, sg, counts, n, hidden, experts, top, s);
}

// counts and cursor: `experts` ints each, zero on entry (cursor is left as the counts).
Q25_EXPORT int q25_moe_sort(const int* topk_idx, const int* counts, int* cursor, int* plan, int* row_pair, int* pair_row, int n_pairs,
                            int experts, int tile, void* stream) {
  if (n_pairs <= 0) return 0;
  const int max_rows = q25_moe_max_rows(n_pairs, experts, tile);
  launch(moe_plan_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, counts, plan, row_pair, experts, tile, max_rows);
  launch(moe_scatter_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0, (cudaStream_t)stream, topk_idx, (const int*)plan, cursor, row_pair,
         pair_row, n_pairs);
  return launch_status();
}

template <bool GATE_UP>
static int moe_grouped_mma(const void* A, const void* W0, const void* W1, void* out, const int* plan, const int* row_pair,
                           const float* topk_w, int n_pairs, int experts, int top, int N, int K, float limit, float alpha, int tile,
                           void* stream) {
  const int tiles = q25_moe_max_rows(n_pairs, experts, tile) / tile;
  if (tile == 16) {
    launch(moe_grouped_mma_kernel<GATE_UP, 16>, dim3((N + 63) / 64, tiles), dim3(128), 0, (cudaStream_t)stream, (const bf16*)A,
           (const bf16*)W0, (const bf16*)W1, out, plan, row_pair, topk_w, experts, top, N, K, limit, alpha);
  } else if (tile == 64) {
    launch(moe_grouped_mma_kernel<GATE_UP, 64>, dim3((N + 63) / 64, tiles), dim3(128), 0, (cudaStream_t)stream, (const bf16*)A,
           (const bf16*)W0, (const bf16*)W1, out, plan, row_pair, topk_w, experts, top, N, K, limit, alpha);
  } else {
    return (int)cudaErrorInvalidValue;
  }
  return launch_status();
}

template <typename T, bool GATE_UP>
static int moe_grouped_fma(const void* A, const void* W0, const void* W1, void* out, const int* plan, const int* row_pair,
                           const float* topk_w, int n_pairs, int experts, int top, int N, int K, float limit, float alpha, int tile,
                           void* stream) {
  if (n_pairs <= 0) return 0;
  // bfloat16 operands whose rows start on 16-byte boundaries go to the tensor cores
  if (sizeof(T) == 2 && K % 8 == 0 && !(((uintptr_t)A | (uintptr_t)W0 | (uintptr_t)W1) & 15))
    return moe_grouped_mma<GATE_UP>(A, W0, W1, out, plan, row_pair, topk_w, n_pairs, experts, top, N, K, limit, alpha, tile, stream);
  const int tiles = q25_moe_max_rows(n_pairs, experts, tile) / tile;
  if (tile == 16) {
    launch(moe_grouped_fma_kernel<T, GATE_UP, 16, 64, 16, 1, 4>, dim3((N + 63) / 64, tiles), dim3(256), 0, (cudaStream_t)stream,
           (const T*)A, (const T*)W0, (const T*)W1, out, plan, row_pair, topk_w, experts, top, N, K, limit, alpha);
  } else if (tile == 64) {
    launch(moe_grouped_fma_kernel<T, GATE_UP, 64, 64, 16, 4, 4>, dim3((N + 63) / 64, tiles), dim3(256), 0, (cudaStream_t)stream,
           (const T*)A, (const T*)W0, (const T*)W1, out, plan, row_pair, topk_w, experts, top, N, K, limit, alpha);
  } else {
    return (int)cudaErrorInvalidValue;
  }
  return launch_status();
}

Q25_EXPORT int q25_moe_gate_up_f32(const void* h, const void* wg, const void* wu, void* act, const int* plan, const int* row_pair,
                                   const float* topk_w, int n_pairs, int experts, int top, int ff, int hidden, float limit,
                                   float alpha, int tile, void* s) {
  return moe_grouped_fma<float, true>(h, wg, wu, act, plan, row_pair, topk_w, n_pairs, experts, top, ff, hidden, limit, alpha, tile, s);
}
Q25_EXPORT int q25_moe_gate_up_bf16(const void* h, const void* wg, const void* wu, void* act, const int* plan, const int* row_pair,
                                    const float* topk_w, int n_pairs, int experts, int top, int ff, int hidden, float limit,
                                    float alpha, int tile, void* s) {
  return moe_grouped_fma<bf16, true>(h, wg, wu, act, plan, row_pair, topk_w, n_pairs, experts, top, ff, hidden, limit, alpha, tile, s);
}
Q25_EXPORT int q25_moe_down_f32(const void* act, const void* wd, void* y, const int* plan, const int* row_pair, int n_pairs,
                                int experts, int top, int hidden, int ff, int tile, void* s) {
  return moe_grouped_fma<float, false>(act, wd, nullptr, y, plan, row_pair, nullptr, n_pairs, experts, top, hidden, ff, 0.f, 0.f, tile, s);
}
Q25_EXPORT int q25_moe_down_bf16(const void* act, const void* wd, void* y, const int* plan, const int* row_pair, int n_pairs,
                                 int experts, int top, int hidden, int ff, int tile, void* s) {
  return moe_grouped_fma<bf16, false>(act, wd, nullptr, y, plan, row_pair, nullptr, n_pairs, experts, top, hidden, ff, 0.f, 0.f, tile, s);
}

template <typename T>
static int moe_combine(const float* y, const int* pair_row, const float* sg, const void* shared, void* out, int n_tokens, int hidden,
                       int top, void* stream) {
  if (n_tokens <= 0) return 0;
  const size_t total = (size_t)n_tokens * hidden;
  size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  launch(moe_combine_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, y, pair_row, sg, (const T*)shared, (T*)out,
         n_tokens, hidden, top);
  return launch_status();
}
Q25_EXPORT int q25_moe_combine_f32(const float* y, const int* pr, const float* sg, const void* sh, void* out, int n, int h, int top, void* s) {
  return moe_combine<float>(y, pr, sg, sh, out, n, h, top, s);
}
Q25_EXPORT int q25_moe_combine_bf16(const float* y, const int* pr, const float* sg, const void* sh, void* out, int n, int h, int top, void* s) {
  return moe_combine<bf16>(y, pr, sg, sh, out, n, h, top, s);
}
