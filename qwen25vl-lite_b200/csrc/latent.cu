// Latent attention keeps one compressed row per token instead of keys and values per head: the
// latent c (RMS-normed, with a weight) followed by one rotated key part that all heads share.  This
// kernel makes that row from the down projection's output and writes it into the token's page slot.
//
//   row[0 .. C)      = x[0 .. C) / sqrt(mean(x[0 .. C)^2) + eps) * w        (statistics in float)
//   row[C .. C + R)  = rotate(x[C .. C + R))                                 (not normed)
//
// The attention kernels then read the row as the single kv head's key (C + R channels) and its first
// C channels as the value.
#include "rotary.cuh"

template <typename T, bool EXACT>
__global__ void latent_store_kernel(const T* __restrict__ x, int x_row, int C, int R, const float* __restrict__ w, float eps,
                                    const float* __restrict__ angles, int half, int layout, T* __restrict__ pages,
                                    const int* __restrict__ kv_slot) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const int tok = blockIdx.x;
  const T* xr = x + (size_t)tok * x_row;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = to_f32(xr[c]);
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = EXACT ? 1.0f / sqrtf(total / (float)C + eps) : rsqrtf(total / (float)C + eps);
  const int slot = kv_slot[tok];
  if (slot < 0) return;
  T* row = pages + (size_t)slot * (C + R);
  for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = from_f32<T>(to_f32(xr[c]) * inv * w[c]);
  const float* ang = angles ? angles + (size_t)tok * half * 2 : nullptr;
  for (int c = threadIdx.x; c < R; c += blockDim.x) row[C + c] = from_f32<T>(rotary_channel<T>(xr + C, c, half, layout, ang));
}

template <typename T, bool EXACT>
static int latent_store(const void* x, int x_row, int C, int R, const float* w, float eps, const float* angles, int half, int layout,
                        void* pages, const int* kv_slot, int n, void* stream) {
  if (n <= 0) return 0;
  if (C <= 0 || R < 0 || 2 * half > R) return (int)cudaErrorInvalidValue;
  launch(latent_store_kernel<T, EXACT>, dim3(n), dim3(128), 0, (cudaStream_t)stream, (const T*)x, x_row, C, R, w, eps, angles, half,
         layout, (T*)pages, kv_slot);
  return launch_status();
}
Q25_EXPORT int q25_latent_store_f32(const void* x, int xr, int C, int R, const float* w, float eps, const float* ang, int half,
                                    int layout, void* pages, const int* slot, int n, void* s) {
  return latent_store<float, true>(x, xr, C, R, w, eps, ang, half, layout, pages, slot, n, s);
}
Q25_EXPORT int q25_latent_store_bf16(const void* x, int xr, int C, int R, const float* w, float eps, const float* ang, int half,
                                     int layout, void* pages, const int* slot, int n, void* s) {
  return latent_store<bf16, false>(x, xr, C, R, w, eps, ang, half, layout, pages, slot, n, s);
}
