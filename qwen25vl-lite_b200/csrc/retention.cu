// Retention: linear attention with a fixed decay per head and neither softmax nor denominator.
// Per head, with q and k rotated by position (rotary.cuh) and k scaled:
//
//   S_t = decay * S_(t-1) + k_t v_t^T        (S: [D, Dv], float, carried from token to token per request)
//   o_t = S_t^T q_t
//   out_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)        (per head; g: a gate of the same size as o)
//
// Everything after the projections is float in both dtypes: the rotation, k's scale, S, o, the unit
// norm and the gate's product; only the result is rounded to the activation dtype.
//
// The kernels walk tokens one after the other, one CTA per (piece of work, head), thread (j, part) owning
// column j of S for a P-th of the rows: retention_rows_kernel with those rows in registers (head sizes
// that 4, 8, 16 or 32 divides), retention_scan_kernel with S in shared memory (any sizes).  Steps of
// single tokens, and short runs, take the walk alone, a CTA per entry.  Long runs are cut into chunks (the host
// plans them): every chunk's own sum of decayed k v^T from zero, all chunks in parallel; a short pass
// that folds the sums onto the request's S in order and leaves each chunk the S before it; then every
// chunk's outputs, again all in parallel.  Twice the arithmetic, and as many CTAs as the run has chunks.
#include "rotary.cuh"

struct RetentionArgs {
  const void* x;          // rows of the projections: q | k | v | g channels at the offsets below
  int x_row, q_off, k_off, v_off, g_off;
  const float* angles;    // [tokens, half, 2] or nullptr
  int half, layout;
  const float* decay;     // [heads]
  float* state;           // [slots, heads, D, Dv]
  const int* cu_q;
  const int* slot_ids;
  void* out;              // [tokens, heads * Dv]
  int heads, D, Dv, P;
  float k_scale, eps;
  // chunked runs
  int s_global;           // the walk with S in shared memory leaves S in global memory instead: heads too large for it
  const int* chunks;      // (entry, first token row, tokens, last of its run) per chunk
  float* sums;            // [chunks, heads, D, Dv]: a chunk's own sum, then the S before the chunk
};

template <typename T>
__device__ __forceinline__ void retention_load_qk(const RetentionArgs& a, int tok, int head, float* q, float* k) {
  const T* row = reinterpret_cast<const T*>(a.x) + (size_t)tok * a.x_row;
  const float* ang = a.angles ? a.angles + (size_t)tok * a.half * 2 : nullptr;
  const T* qh = row + a.q_off + (size_t)head * a.D;
  const T* kh = row + a.k_off + (size_t)head * a.D;
  for (int c = threadIdx.x; c < a.D; c += blockDim.x) {
    q[c] = rotary_channel<T>(qh, c, a.half, a.layout, ang);
    k[c] = rotary_channel<T>(kh, c, a.half, a.layout, ang) * a.k_scale;
  }
}

// o (one value per thread of part 0, column j) -> unit RMS over the head, times silu(g), stored.
template <typename T>
__device__ __forceinline__ void retention_finish(const RetentionArgs& a, int tok, int head, int j, bool owner, float o, float* scratch) {
  const float total = block_sum(owner ? o * o : 0.f, scratch);
  if (owner) {
    const T* row = reinterpret_cast<const T*>(a.x) + (size_t)tok * a.x_row;
    const float g = to_f32(row[a.g_off + (size_t)head * a.Dv + j]);
    const float inv = 1.0f / sqrtf(total / (float)a.Dv + a.eps);
    reinterpret_cast<T*>(a.out)[(size_t)tok * a.heads * a.Dv + (size_t)head * a.Dv + j] = from_f32<T>(o * inv * (g / (1.0f + expf(-g))));
  }
}

// MODE 0: blockIdx.x is an entry; its tokens from the request's state, which moves on (entries of more
//         than `long_from` tokens are left to the chunked kernels; 0: none are).
// MODE 1: blockIdx.x is a chunk (entry, first token row, tokens, last of its run); S starts at zero,
//         nothing is put out, and S goes to sums[chunk] (the last chunk of a run is skipped: nobody
//         reads its sum).
// MODE 2: blockIdx.x is a chunk; S starts from sums[chunk] (by then the request's S before the chunk),
//         the outputs are written, and the run's last chunk leaves S in the request's state.
template <typename T, int MODE>
__global__ void retention_scan_kernel(RetentionArgs a, int long_from) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float ret_smem[];
  const int D = a.D, Dv = a.Dv, P = a.P;
  float* q = ret_smem + (a.s_global ? 0 : (size_t)D * Dv);       // [D]
  float* k = q + D;                    // [D]
  float* part = k + D;                 // [P][Dv]
  float* scratch = part + P * Dv;      // [32]
  const int head = blockIdx.y;
  int entry, first, last;
  bool is_last = true;
  if (MODE == 0) {
    entry = blockIdx.x;
    first = a.cu_q[entry];
    last = a.cu_q[entry + 1];
    if (long_from > 0 && last - first > long_from) return;
  } else {
    const int* c = a.chunks + 4 * blockIdx.x;
    entry = c[0];
    first = c[1];
    last = first + c[2];
    is_last = c[3] != 0;
    if (MODE == 1 && is_last) return;
  }
  const size_t SZ = (size_t)D * Dv;
  float* Sreq = a.state + ((size_t)a.slot_ids[entry] * a.heads + head) * SZ;
  float* Ssum = MODE == 0 ? nullptr : a.sums + ((size_t)blockIdx.x * a.heads + head) * SZ;
  const float* Sin = MODE == 0 ? Sreq : Ssum;
  // [D][Dv]: in shared memory, or where it lies in global memory (an element is only ever touched by its owner thread)
  float* S = a.s_global ? (MODE == 0 ? Sreq : Ssum) : ret_smem;
  if (!a.s_global || MODE == 1)
    for (int x = threadIdx.x; x < D * Dv; x += blockDim.x) S[x] = MODE == 1 ? 0.f : Sin[x];
  const bool active = threadIdx.x < Dv * P;       // the CTA is filled up to whole warps; the extra threads only copy
  const int j = threadIdx.x % Dv, p = active ? (int)threadIdx.x / Dv : -1;
  const int rows = D / P, i0 = p * rows;
  const float decay = a.decay[head];
  for (int tok = first; tok < last; ++tok) {
    __syncthreads();                   // S loaded / the token before is done with q, k and part
    retention_load_qk<T>(a, tok, head, q, k);
    __syncthreads();
    if (active) {
      const float vj = to_f32(reinterpret_cast<const T*>(a.x)[(size_t)tok * a.x_row + a.v_off + (size_t)head * Dv + j]);
      float acc = 0.f;
      for (int i = i0; i < i0 + rows; ++i) {
        const float s = fmaf(decay, S[i * Dv + j], k[i] * vj);
        S[i * Dv + j] = s;
        acc = fmaf(s, q[i], acc);
      }
      part[p * Dv + j] = acc;
    }
    if (MODE == 1) continue;
    __syncthreads();
    float o = 0.f;
    if (p == 0)
      for (int pp = 0; pp < P; ++pp) o += part[pp * Dv + j];
    retention_finish<T>(a, tok, head, j, p == 0, o, scratch);
  }
  __syncthreads();
  float* Sout = MODE == 1 ? Ssum : (is_last ? Sreq : nullptr);
  if (Sout && Sout != S)
    for (int x = threadIdx.x; x < D * Dv; x += blockDim.x) Sout[x] = S[x];
}

// Between the two chunked passes: for every run (entry, first chunk, chunks) and head, element by
// element, the chunks' own sums are folded onto the request's S in order, and every chunk's slot is
// left holding the S before it: S_before(c + 1) = decay^tokens(c) * S_before(c) + sum(c).
__global__ void retention_fold_kernel(RetentionArgs a, const int* __restrict__ runs) {
  pdl_trigger();
  pdl_wait();
  const int* r = runs + 3 * blockIdx.x;
  const int entry = r[0], c0 = r[1], n = r[2], head = blockIdx.y;
  const size_t SZ = (size_t)a.D * a.Dv;
  const float* Sreq = a.state + ((size_t)a.slot_ids[entry] * a.heads + head) * SZ;
  const float decay = a.decay[head];
  constexpr int B = 8;                                       // sums in flight per thread
  for (size_t x = (size_t)blockIdx.z * blockDim.x + threadIdx.x; x < SZ; x += (size_t)gridDim.z * blockDim.x) {
    float s = Sreq[x];
    for (int b0 = 0; b0 < n; b0 += B) {
      float own[B];
#pragma unroll
      for (int i = 0; i < B; ++i) {
        const int c = c0 + b0 + i;
        own[i] = b0 + i + 1 < n ? __ldcg(a.sums + ((size_t)c * a.heads + head) * SZ + x) : 0.f;   // the last chunk left none
      }
#pragma unroll
      for (int i = 0; i < B; ++i) {
        if (b0 + i < n) {
          const int c = c0 + b0 + i;
          a.sums[((size_t)c * a.heads + head) * SZ + x] = s;
          s = fmaf(powf(decay, (float)a.chunks[4 * c + 2]), s, own[i]);
        }
      }
    }
  }
}

// The same walk with the thread's rows of S in registers, for head sizes that ROWS divides: thread
// (j, part) owns rows part * ROWS .. of column j.  Four more warps only load: they rotate and scale the
// keys and queries of the next RET_TB tokens into one half of a double buffer (with the values) while
// the others work through the half before, so that no trip to memory stands in the walk; the CTA meets
// once per RET_TB tokens.  The raw outputs of up to `group` tokens wait in shared memory, each part's
// share apart, beside the tokens' gates (the loaders bring them with the values), and are normalised and
// gated afterwards, a warp per token, with no trip to memory but the store.  mode as MODE above.
#define RET_TB 4
#define RET_LOADERS 128
#define RET_MAX_THREADS 640   // 512 that compute and the loaders: registers for 32 rows of S a thread

template <typename T, int ROWS>
__global__ void __launch_bounds__(RET_MAX_THREADS) retention_rows_kernel(RetentionArgs a, int mode, int long_from, int group) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float ret_smem[];
  const int D = a.D, Dv = a.Dv, P = D / ROWS;
  float2* kq = reinterpret_cast<float2*>(ret_smem);   // [2][RET_TB][D]: (scaled rotated key, rotated query)
  float* vs = ret_smem + 2 * 2 * RET_TB * D;          // [2][RET_TB][Dv]
  float* obuf = vs + 2 * RET_TB * Dv;                 // [P][group][Dv]
  float* gs = obuf + (size_t)P * group * Dv;          // [group][Dv]: the tokens' gates, brought by the loaders with the values
  const int head = blockIdx.y;
  int entry, first, last;
  bool is_last = true;
  if (mode == 0) {
    entry = blockIdx.x;
    first = a.cu_q[entry];
    last = a.cu_q[entry + 1];
    if (long_from > 0 && last - first > long_from) return;
  } else {
    const int* c = a.chunks + 4 * blockIdx.x;
    entry = c[0];
    first = c[1];
    last = first + c[2];
    is_last = c[3] != 0;
    if (mode == 1 && is_last) return;
  }
  const size_t SZ = (size_t)D * Dv;
  float* Sreq = a.state + ((size_t)a.slot_ids[entry] * a.heads + head) * SZ;
  float* Ssum = mode == 0 ? nullptr : a.sums + ((size_t)blockIdx.x * a.heads + head) * SZ;
  const float* Sin = mode == 0 ? Sreq : Ssum;
  const int n_compute = blockDim.x - RET_LOADERS;
  const bool loader = (int)threadIdx.x >= n_compute;
  const int ltid = (int)threadIdx.x - n_compute;
  const bool active = !loader && (int)threadIdx.x < Dv * P;
  const int j = threadIdx.x % Dv, p = threadIdx.x / Dv, i0 = p * ROWS;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) s[r] = active && mode != 1 ? Sin[(size_t)(i0 + r) * Dv + j] : 0.f;
  const float decay = a.decay[head];
  const T* X = reinterpret_cast<const T*>(a.x);

  for (int g0 = first; g0 < last; g0 += group) {
    const int cnt = min(group, last - g0), nb = (cnt + RET_TB - 1) / RET_TB;
    // The loaders' part.  A loader keeps its channel and walks the batch's tokens, so that nothing is
    // divided and all loads of a batch are asked for before any is used: one trip to memory a batch.
    auto fill = [&](int b) {
      const int t0 = g0 + b * RET_TB, nt = min(RET_TB, g0 + cnt - t0), base = (b & 1) * RET_TB;
      const int half = a.angles ? a.half : 0, turned = 2 * half;
      for (int c = ltid; c < (D > Dv ? D : Dv); c += RET_LOADERS) {
        int iu = c, iv = c, i = 0;
        bool second = false;
        if (c < turned) {                                     // the pair (u, v) this channel belongs to, and which of the two it is
          if (a.layout == ROTARY_INTERLEAVED) { i = c >> 1; iu = 2 * i; iv = iu + 1; second = c & 1; }
          else { second = c >= half; i = second ? c - half : c; iu = i; iv = i + half; }
        }
        const bool is_k = c < D, is_v = c < Dv, turn = c < turned;
        // Every load of the batch is asked for before the first is used: the addresses are clamped to
        // valid ones instead of guarded (a branch would put the first use, and its wait, between the
        // loads), and the values stay as they were loaded until the second loop.
        const int cv = is_v ? c : 0, ck_u = is_k ? iu : 0, ck_v = is_k ? iv : 0, ia = turn ? i : 0;
        const T* row0 = X + (size_t)t0 * a.x_row;
        const float* ang0 = a.angles ? a.angles + ((size_t)t0 * half + ia) * 2 : nullptr;
        T raw[RET_TB], gat[RET_TB], ku[RET_TB], kv[RET_TB], qu[RET_TB], qv[RET_TB];
        float2 cssn[RET_TB];
#pragma unroll
        for (int tt = 0; tt < RET_TB; ++tt) {
          const int tc = tt < nt ? tt : nt - 1;
          const T* row = row0 + (size_t)tc * a.x_row;
          raw[tt] = row[a.v_off + (size_t)head * Dv + cv];
          gat[tt] = row[a.g_off + (size_t)head * Dv + cv];
          ku[tt] = row[a.k_off + (size_t)head * D + ck_u];
          kv[tt] = row[a.k_off + (size_t)head * D + ck_v];
          qu[tt] = row[a.q_off + (size_t)head * D + ck_u];
          qv[tt] = row[a.q_off + (size_t)head * D + ck_v];
          cssn[tt] = ang0 ? *reinterpret_cast<const float2*>(ang0 + (size_t)tc * half * 2) : make_float2(1.f, 0.f);
        }
#pragma unroll
        for (int tt = 0; tt < RET_TB; ++tt) {
          if (tt < nt) {
            if (is_v) {
              vs[(base + tt) * Dv + c] = to_f32(raw[tt]);
              if (mode != 1) gs[(size_t)(b * RET_TB + tt) * Dv + c] = to_f32(gat[tt]);
            }
            if (is_k) {
              const float u = to_f32(ku[tt]), v = to_f32(kv[tt]), uq = to_f32(qu[tt]), vq = to_f32(qv[tt]);
              const float cs = cssn[tt].x, sn = cssn[tt].y;
              float kk, qq;
              if (!turn) { kk = u; qq = uq; }
              else if (second) { kk = fmaf(v, cs, u * sn); qq = fmaf(vq, cs, uq * sn); }
              else { kk = fmaf(u, cs, -v * sn); qq = fmaf(uq, cs, -vq * sn); }
              kq[(base + tt) * D + c] = make_float2(kk * a.k_scale, mode == 1 ? 0.f : qq);
            }
          }
        }
      }
    };
    if (loader) fill(0);
    __syncthreads();
    for (int b = 0; b < nb; ++b) {
      if (loader) {
        if (b + 1 < nb) fill(b + 1);
      } else if (active) {
        const int t_end = min(cnt, (b + 1) * RET_TB);
        for (int t = b * RET_TB; t < t_end; ++t) {
          const int slot = (b & 1) * RET_TB + (t - b * RET_TB);
          const float vj = vs[slot * Dv + j];
          const float4* row = reinterpret_cast<const float4*>(kq + slot * D + i0);       // two rows a load
          float acc = 0.f;
#pragma unroll
          for (int r = 0; r < ROWS; r += 2) {
            const float4 x = row[r >> 1];
            s[r] = fmaf(decay, s[r], x.x * vj);
            acc = fmaf(s[r], x.y, acc);
            s[r + 1] = fmaf(decay, s[r + 1], x.z * vj);
            acc = fmaf(s[r + 1], x.w, acc);
          }
          if (mode != 1) obuf[((size_t)p * group + t) * Dv + j] = acc;
        }
      }
      __syncthreads();
    }
    if (mode != 1) {
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
      for (int t = warp; t < cnt; t += nwarps) {
        const size_t tok = (size_t)(g0 + t);
        float ss = 0.f;
        for (int jj = lane; jj < Dv; jj += 32) {
          float o = 0.f;
          for (int pp = 0; pp < P; ++pp) o += obuf[((size_t)pp * group + t) * Dv + jj];
          obuf[(size_t)t * Dv + jj] = o;                                  // part 0's place now holds the sum (this lane's own element)
          ss = fmaf(o, o, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
        T* orow = reinterpret_cast<T*>(a.out) + tok * a.heads * Dv + (size_t)head * Dv;
        for (int jj = lane; jj < Dv; jj += 32) {
          const float g = gs[(size_t)t * Dv + jj];
          orow[jj] = from_f32<T>(obuf[(size_t)t * Dv + jj] * inv * (g / (1.0f + expf(-g))));
        }
      }
      __syncthreads();                                 // the outputs' places are free for the next tokens
    }
  }
  float* Sout = mode == 1 ? Ssum : (is_last ? Sreq : nullptr);
  if (Sout && active) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) Sout[(size_t)(i0 + r) * Dv + j] = s[r];
  }
}

// How many ways the rows of S are cut among the threads of a column: the most that divides D and
// keeps the CTA within 256 threads.
static int retention_parts(int D, int Dv) {
  int P = 1;
  for (int c = 2; c * Dv <= 256 && c <= D; ++c)
    if (D % c == 0) P = c;
  return P;
}

// chunks: n_chunks x (entry, first token row, tokens, last of its run) for the entries of more than
// `long_from` tokens, runs: n_runs x (entry, first chunk, chunks), sums: n_chunks * heads * D * Dv floats;
// all entries up to long_from tokens (every entry when there are no chunks) take the plain scan.
template <typename T>
static int retention_run(const void* x, int x_row, int q_off, int k_off, int v_off, int g_off, const float* angles, int half, int layout,
                         const float* decay, float* state, const int* cu_q, const int* slot_ids, void* out, int n_seqs, int heads,
                         int D, int Dv, float k_scale, float eps, const int* chunks, int n_chunks, const int* runs, int n_runs,
                         float* sums, int long_from, int scan_too, void* stream) {
  if (n_seqs <= 0) return 0;
  if (D <= 0 || Dv <= 0 || Dv > 1024 || 2 * half > D || (n_chunks > 0 && (!chunks || !runs || !sums || n_runs <= 0 || long_from <= 0)))
    return (int)cudaErrorInvalidValue;
  RetentionArgs a;
  a.x = x; a.x_row = x_row; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
  a.angles = angles; a.half = half; a.layout = layout; a.decay = decay; a.state = state; a.cu_q = cu_q; a.slot_ids = slot_ids;
  a.out = out; a.heads = heads; a.D = D; a.Dv = Dv; a.P = retention_parts(D, Dv); a.k_scale = k_scale; a.eps = eps;
  a.chunks = chunks; a.sums = sums; a.s_global = 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int per = (int)(((size_t)D * Dv + 255) / 256);
  const dim3 fold_grid(n_runs > 0 ? n_runs : 1, heads, per < 64 ? per : 64);
  // S in registers where the head size has a divisor among the row counts the kernel is built for
  int rows = 0;
  for (int r = 32; r >= 4; r >>= 1)
    if (D % r == 0) { rows = r; break; }
  if (rows) {
    const int P = D / rows, compute = (Dv * P + 31) / 32 * 32;
    int group = 16384 / (P * Dv);
    group = group > 64 ? 64 : (group < 1 ? 1 : group);
    const size_t smem = ((size_t)2 * 2 * RET_TB * D + (size_t)2 * RET_TB * Dv + (size_t)(P + 1) * group * Dv) * sizeof(float);
    if (compute + RET_LOADERS <= RET_MAX_THREADS && smem <= 200 * 1024) {
      void (*kernel)(RetentionArgs, int, int, int) =
          rows == 32 ? retention_rows_kernel<T, 32> : rows == 16 ? retention_rows_kernel<T, 16>
          : rows == 8 ? retention_rows_kernel<T, 8> : retention_rows_kernel<T, 4>;
      if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      const dim3 block(compute + RET_LOADERS);
      if (scan_too) launch(kernel, dim3(n_seqs, heads), block, smem, s, a, 0, n_chunks > 0 ? long_from : 0, group);
      if (n_chunks > 0) {
        launch(kernel, dim3(n_chunks, heads), block, smem, s, a, 1, 0, group);
        launch(retention_fold_kernel, fold_grid, dim3(256), 0, s, a, runs);
        launch(kernel, dim3(n_chunks, heads), block, smem, s, a, 2, 0, group);
      }
      return launch_status();
    }
  }
  // any other sizes: S in shared memory
  size_t smem = ((size_t)D * Dv + 2 * D + (size_t)a.P * Dv + 32) * sizeof(float);
  if (smem > 200 * 1024) {                       // a head whose S does not fit: it stays in global memory, walked in place
    a.s_global = 1;
    smem = ((size_t)2 * D + (size_t)a.P * Dv + 32) * sizeof(float);
  }
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(retention_scan_kernel<T, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(retention_scan_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(retention_scan_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 block((Dv * a.P + 31) / 32 * 32);
  if (scan_too) launch(retention_scan_kernel<T, 0>, dim3(n_seqs, heads), block, smem, s, a, n_chunks > 0 ? long_from : 0);
  if (n_chunks > 0) {
    launch(retention_scan_kernel<T, 1>, dim3(n_chunks, heads), block, smem, s, a, 0);
    launch(retention_fold_kernel, fold_grid, dim3(256), 0, s, a, runs);
    launch(retention_scan_kernel<T, 2>, dim3(n_chunks, heads), block, smem, s, a, 0);
  }
  return launch_status();
}

Q25_EXPORT int q25_retention_f32(const void* x, int xr, int qo, int ko, int vo, int go, const float* ang, int half, int layout,
                                 const float* decay, float* state, const int* cu, const int* slots, void* out, int n_seqs, int heads,
                                 int D, int Dv, float k_scale, float eps, const int* chunks, int n_chunks, const int* runs, int n_runs,
                                 float* sums, int long_from, int scan_too, void* s) {
  return retention_run<float>(x, xr, qo, ko, vo, go, ang, half, layout, decay, state, cu, slots, out, n_seqs, heads, D, Dv, k_scale, eps,
                              chunks, n_chunks, runs, n_runs, sums, long_from, scan_too, s);
}
Q25_EXPORT int q25_retention_bf16(const void* x, int xr, int qo, int ko, int vo, int go, const float* ang, int half, int layout,
                                  const float* decay, float* state, const int* cu, const int* slots, void* out, int n_seqs, int heads,
                                  int D, int Dv, float k_scale, float eps, const int* chunks, int n_chunks, const int* runs, int n_runs,
                                  float* sums, int long_from, int scan_too, void* s) {
  return retention_run<bf16>(x, xr, qo, ko, vo, go, ang, half, layout, decay, state, cu, slots, out, n_seqs, heads, D, Dv, k_scale, eps,
                             chunks, n_chunks, runs, n_runs, sums, long_from, scan_too, s);
}
