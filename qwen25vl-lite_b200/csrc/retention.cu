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
// retention_scan_kernel walks an entry's tokens one after the other with S in shared memory: one CTA
// per (entry, head), Dv * P threads: thread (j, part) owns column j of S for a P-th of the rows.
// Steps of single tokens, and short runs, take it alone.  Long runs are cut into chunks of
// RET_CHUNK tokens (retention_chunk_*): every chunk's own sum of decayed k v^T in parallel, a short
// pass that folds them onto the request's S in order, and then every chunk's outputs in parallel
// from the S before it and the chunk's own keys.
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

template <typename T>
__global__ void retention_scan_kernel(RetentionArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float ret_smem[];
  const int D = a.D, Dv = a.Dv, P = a.P;
  float* S = ret_smem;                 // [D][Dv]
  float* q = S + (size_t)D * Dv;       // [D]
  float* k = q + D;                    // [D]
  float* part = k + D;                 // [P][Dv]
  float* scratch = part + P * Dv;      // [32]
  const int entry = blockIdx.x, head = blockIdx.y;
  const int first = a.cu_q[entry], last = a.cu_q[entry + 1];
  float* Sg = a.state + ((size_t)a.slot_ids[entry] * a.heads + head) * D * Dv;
  for (int x = threadIdx.x; x < D * Dv; x += blockDim.x) S[x] = Sg[x];
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
    __syncthreads();
    float o = 0.f;
    if (p == 0)
      for (int pp = 0; pp < P; ++pp) o += part[pp * Dv + j];
    retention_finish<T>(a, tok, head, j, p == 0, o, scratch);
  }
  __syncthreads();
  for (int x = threadIdx.x; x < D * Dv; x += blockDim.x) Sg[x] = S[x];
}

// How many ways the rows of S are cut among the threads of a column: the most that divides D and
// keeps the CTA within 256 threads.
static int retention_parts(int D, int Dv) {
  int P = 1;
  for (int c = 2; c * Dv <= 256 && c <= D; ++c)
    if (D % c == 0) P = c;
  return P;
}

template <typename T>
static int retention_scan(const void* x, int x_row, int q_off, int k_off, int v_off, int g_off, const float* angles, int half, int layout,
                          const float* decay, float* state, const int* cu_q, const int* slot_ids, void* out, int n_seqs, int heads,
                          int D, int Dv, float k_scale, float eps, void* stream) {
  if (n_seqs <= 0) return 0;
  if (D <= 0 || Dv <= 0 || Dv > 1024 || 2 * half > D) return (int)cudaErrorInvalidValue;
  RetentionArgs a;
  a.x = x; a.x_row = x_row; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
  a.angles = angles; a.half = half; a.layout = layout; a.decay = decay; a.state = state; a.cu_q = cu_q; a.slot_ids = slot_ids;
  a.out = out; a.heads = heads; a.D = D; a.Dv = Dv; a.P = retention_parts(D, Dv); a.k_scale = k_scale; a.eps = eps;
  a.chunks = nullptr; a.sums = nullptr;
  const size_t smem = ((size_t)D * Dv + 2 * D + (size_t)a.P * Dv + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(retention_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(retention_scan_kernel<T>, dim3(n_seqs, heads), dim3((Dv * a.P + 31) / 32 * 32), smem, (cudaStream_t)stream, a);
  return launch_status();
}

Q25_EXPORT int q25_retention_scan_f32(const void* x, int xr, int qo, int ko, int vo, int go, const float* ang, int half, int layout,
                                      const float* decay, float* state, const int* cu, const int* slots, void* out, int n_seqs, int heads,
                                      int D, int Dv, float k_scale, float eps, void* s) {
  return retention_scan<float>(x, xr, qo, ko, vo, go, ang, half, layout, decay, state, cu, slots, out, n_seqs, heads, D, Dv, k_scale, eps, s);
}
Q25_EXPORT int q25_retention_scan_bf16(const void* x, int xr, int qo, int ko, int vo, int go, const float* ang, int half, int layout,
                                       const float* decay, float* state, const int* cu, const int* slots, void* out, int n_seqs, int heads,
                                       int D, int Dv, float k_scale, float eps, void* s) {
  return retention_scan<bf16>(x, xr, qo, ko, vo, go, ang, half, layout, decay, state, cu, slots, out, n_seqs, heads, D, Dv, k_scale, eps, s);
}
