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
// retention_scan_kernel walks tokens one after the other with S in shared memory: one CTA per (piece of
// work, head), Dv * P threads: thread (j, part) owns column j of S for a P-th of the rows.  Steps of
// single tokens, and short runs, take it alone, a CTA per entry.  Long runs are cut into chunks (the host
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
  const int* chunks;      // (entry, first token of the chunk within the entry) pairs
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
  float* S = ret_smem;                 // [D][Dv]
  float* q = S + (size_t)D * Dv;       // [D]
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
  if (Sout)
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
  for (size_t x = (size_t)blockIdx.z * blockDim.x + threadIdx.x; x < SZ; x += (size_t)gridDim.z * blockDim.x) {
    float s = Sreq[x];
    for (int c = c0; c < c0 + n; ++c) {
      float* slot = a.sums + ((size_t)c * a.heads + head) * SZ + x;
      const float own = c + 1 < c0 + n ? *slot : 0.f;      // the last chunk left none
      *slot = s;
      s = fmaf(powf(decay, (float)a.chunks[4 * c + 2]), s, own);
    }
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
  a.chunks = chunks; a.sums = sums;
  const size_t smem = ((size_t)D * Dv + 2 * D + (size_t)a.P * Dv + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(retention_scan_kernel<T, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(retention_scan_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(retention_scan_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 block((Dv * a.P + 31) / 32 * 32);
  cudaStream_t s = (cudaStream_t)stream;
  if (scan_too) launch(retention_scan_kernel<T, 0>, dim3(n_seqs, heads), block, smem, s, a, n_chunks > 0 ? long_from : 0);
  if (n_chunks > 0) {
    launch(retention_scan_kernel<T, 1>, dim3(n_chunks, heads), block, smem, s, a, 0);
    const int per = (int)(((size_t)D * Dv + 255) / 256);
    launch(retention_fold_kernel, dim3(n_runs, heads, per < 8 ? per : 8), dim3(256), 0, s, a, runs);
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
