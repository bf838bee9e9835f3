// Softmax attention over the paged cache with a bias that grows with distance, a sliding window
// beside which the first tokens of the request stay visible, a scale of its own, and values whose
// size may differ from the keys'.  No rotation: positions enter through the bias alone.
//
//   score(i, j) = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))        (r1 == nullptr: no bias)
//   query i sees key j when j <= i and (i - j < window or j < keep_first)       (window 0: all j <= i)
//   o_i = softmax_j(score) v_j;  query head h reads kv head h / (nq / nkv)
//
// and the write of a step's keys and values into their pages, where the values may first be mixed
// with those another layer computed for the same token: v <- (1 - mix) v + mix v_other.
//
// This file holds the general kernels (float or bfloat16, any sizes up to 256): one warp per
// (token, query head); keys are walked in tiles of 32 aligned to the absolute key index, first the
// kept tokens that the window has left behind, then the window; scores, bias and softmax in float.
// The order of every sum depends on the query's position alone.
#include "common.cuh"

#define BATT_WARPS 4
#define BATT_MAX_D 256

template <typename T>
__global__ void biased_attention_generic_kernel(
    const T* __restrict__ qkv, int qkv_stride, T* __restrict__ out, const T* __restrict__ kpages,
    const T* __restrict__ vpages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ token_seq, const int* __restrict__ cu_q, const int* __restrict__ q_start_pos,
    int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int window, int keep_first, float scale,
    const float* __restrict__ r1, const float* __restrict__ r2) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char att_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t per_warp = (size_t)(dk + 32) * sizeof(float) + 32 * sizeof(size_t);
  unsigned char* base = att_smem + warp * per_warp;
  size_t* voff = reinterpret_cast<size_t*>(base);
  float* qs = reinterpret_cast<float*>(base + 32 * sizeof(size_t));
  float* ps = qs + dk;

  const long long item = (long long)blockIdx.x * BATT_WARPS + warp;
  if (item >= (long long)n_tokens * nq) return;
  const int token = (int)(item / nq), head = (int)(item % nq);
  const int kvh = head / (nq / nkv);
  const int seq = token_seq[token];
  if (seq < 0) return;
  const int p = q_start_pos[seq] + token - cu_q[seq];
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (lo <= keep_first) lo = 0;                       // the kept tokens and the window touch: one range
  const int kept = lo > 0 ? keep_first : 0;           // keys [0, kept) and [lo, p]
  const float b1 = r1 ? r1[head] : 0.f, b2 = r1 ? r2[head] : 0.f;

  const T* q = qkv + (size_t)token * qkv_stride + (size_t)head * dk;
  for (int c = lane; c < dk; c += 32) qs[c] = to_f32(q[c]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[BATT_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < BATT_MAX_D / 32; ++i) acc[i] = 0.f;

  const int* table = block_table + (size_t)seq * table_width;
  for (int range = 0; range < 2; ++range) {
    const int first = range == 0 ? 0 : lo, last = range == 0 ? kept - 1 : p;
    for (int t0 = first & ~31; t0 <= last; t0 += 32) {
      const int key = t0 + lane;
      const bool valid = key >= first && key <= last;
      float s = -INFINITY;
      size_t off = 0;
      if (valid) {
        const int page = table[key / page_size];
        const size_t row = ((size_t)page * nkv + kvh) * page_size + (key % page_size);
        off = row * dv;
        const T* kr = kpages + row * dk;
        float dot = 0.f;
        for (int c = 0; c < dk; ++c) dot = fmaf(qs[c], to_f32(kr[c]), dot);
        s = dot * scale;
        if (r1) s -= b1 * log1pf(b2 * (float)(p - key));
      }
      const float m_new = fmaxf(m, warp_max(s));  // finite: every tile holds at least one valid key
      const float pexp = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);          // first tile: exp(-inf) = 0
      l = l * corr + warp_sum(pexp);
      m = m_new;
      ps[lane] = pexp;
      voff[lane] = off;
      __syncwarp();
      const int kmax = min(32, last - t0 + 1);
      const int kmin = max(0, first - t0);
#pragma unroll
      for (int i = 0; i < BATT_MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) {
          float a = acc[i] * corr;
          for (int kk = kmin; kk < kmax; ++kk) a = fmaf(ps[kk], to_f32(vpages[voff[kk] + c]), a);
          acc[i] = a;
        }
      }
      __syncwarp();
    }
  }
  T* o = out + (size_t)token * nq * dv + (size_t)head * dv;
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < BATT_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) o[c] = from_f32<T>(acc[i] * inv_l);
  }
}

// A step's keys and values into their pages.  qkv rows hold nq*dk query, nkv*dk key and nkv*dv value
// channels.  v_other (row stride ld_other, nkv*dv channels a row; nullptr: none): the values that
// another layer computed for the same tokens, mixed in before the write; the mixed values also
// replace the row's own (the layers that follow may ask for them).
template <typename T>
__global__ void kv_store_mix_kernel(T* __restrict__ qkv, int qkv_stride, const T* __restrict__ v_other, int ld_other, float mix,
                                    T* __restrict__ kpages, T* __restrict__ vpages, const int* __restrict__ kv_slot, int n_tokens,
                                    int nq, int nkv, int dk, int dv, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int slot = kv_slot[n];
  T* row = qkv + (size_t)n * qkv_stride;
  const int k_off = nq * dk, v_off = (nq + nkv) * dk;
  const int page = slot / page_size, in_page = slot % page_size;
  for (int c = threadIdx.x; c < nkv * dk; c += blockDim.x) {
    const int h = c / dk, e = c % dk;
    if (slot >= 0) kpages[(((size_t)page * nkv + h) * page_size + in_page) * dk + e] = row[k_off + c];
  }
  for (int c = threadIdx.x; c < nkv * dv; c += blockDim.x) {
    const int h = c / dv, e = c % dv;
    T v = row[v_off + c];
    if (v_other) {
      v = from_f32<T>(fmaf(mix, to_f32(v_other[(size_t)n * ld_other + c]), (1.0f - mix) * to_f32(v)));
      row[v_off + c] = v;
    }
    if (slot >= 0) vpages[(((size_t)page * nkv + h) * page_size + in_page) * dv + e] = v;
  }
}

template <typename T>
static int biased_attention_generic(const void* qkv, int qkv_stride, void* out, const void* kpages, const void* vpages,
                                    const int* block_table, int table_width, const int* token_seq, const int* cu_q,
                                    const int* q_start_pos, int n_tokens, int nq, int nkv, int dk, int dv, int page_size,
                                    int window, int keep_first, float scale, const float* r1, const float* r2, void* stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dv > BATT_MAX_D || dk > 4096 || nkv <= 0 || nq % nkv || window < 0 || keep_first < 0)
    return (int)cudaErrorInvalidValue;
  const long long items = (long long)n_tokens * nq;
  const unsigned blocks = (unsigned)((items + BATT_WARPS - 1) / BATT_WARPS);
  const size_t smem = BATT_WARPS * ((size_t)(dk + 32) * sizeof(float) + 32 * sizeof(size_t));
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(biased_attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(biased_attention_generic_kernel<T>, dim3(blocks), dim3(BATT_WARPS * 32), smem, (cudaStream_t)stream, (const T*)qkv,
         qkv_stride, (T*)out, (const T*)kpages, (const T*)vpages, block_table, table_width, token_seq, cu_q, q_start_pos, n_tokens,
         nq, nkv, dk, dv, page_size, window, keep_first, scale, r1, r2);
  return launch_status();
}

template <typename T>
static int kv_store_mix(void* qkv, int qkv_stride, const void* v_other, int ld_other, float mix, void* kpages, void* vpages,
                        const int* kv_slot, int n_tokens, int nq, int nkv, int dk, int dv, int page_size, void* stream) {
  if (n_tokens <= 0) return 0;
  launch(kv_store_mix_kernel<T>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (T*)qkv, qkv_stride, (const T*)v_other, ld_other,
         mix, (T*)kpages, (T*)vpages, kv_slot, n_tokens, nq, nkv, dk, dv, page_size);
  return launch_status();
}

Q25_EXPORT int q25_biased_attention_generic_f32(const void* qkv, int qs, void* out, const void* kp, const void* vp, const int* bt,
                                                int tw, const int* ts, const int* cu, const int* sp, int n, int nq, int nkv, int dk,
                                                int dv, int ps, int window, int keep, float scale, const float* r1, const float* r2,
                                                void* s) {
  return biased_attention_generic<float>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, dk, dv, ps, window, keep, scale, r1, r2, s);
}
Q25_EXPORT int q25_biased_attention_generic_bf16(const void* qkv, int qs, void* out, const void* kp, const void* vp, const int* bt,
                                                 int tw, const int* ts, const int* cu, const int* sp, int n, int nq, int nkv, int dk,
                                                 int dv, int ps, int window, int keep, float scale, const float* r1, const float* r2,
                                                 void* s) {
  return biased_attention_generic<bf16>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, dk, dv, ps, window, keep, scale, r1, r2, s);
}
Q25_EXPORT int q25_kv_store_mix_f32(void* qkv, int qs, const void* vo, int ldo, float mix, void* kp, void* vp, const int* slot, int n,
                                    int nq, int nkv, int dk, int dv, int ps, void* s) {
  return kv_store_mix<float>(qkv, qs, vo, ldo, mix, kp, vp, slot, n, nq, nkv, dk, dv, ps, s);
}
Q25_EXPORT int q25_kv_store_mix_bf16(void* qkv, int qs, const void* vo, int ldo, float mix, void* kp, void* vp, const int* slot, int n,
                                     int nq, int nkv, int dk, int dv, int ps, void* s) {
  return kv_store_mix<bf16>(qkv, qs, vo, ldo, mix, kp, vp, slot, n, nq, nkv, dk, dv, ps, s);
}
