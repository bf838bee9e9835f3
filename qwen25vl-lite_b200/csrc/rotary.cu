// Rotary position encoding on one axis of positions, for any part of a head and either pairing of
// channels (rotary.cuh).  The angles of a step are computed once, in float from the integer
// positions and a table of frequencies that the host prepared (any scaling of the frequencies is in
// that table; a magnitude multiplies cos and sin), and every layer that shares the table reads them.
#include "rotary.cuh"

// out[n][i] = (cos, sin)(positions[n] * inv_freq[i]) * magnitude
__global__ void rotary_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float magnitude,
                                     float* __restrict__ out, int n, int half) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n * half;
  for (size_t x = (size_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (size_t)gridDim.x * blockDim.x) {
    const int tok = (int)(x / half), i = (int)(x % half);
    float sn, cs;
    sincosf((float)positions[tok] * inv_freq[i], &sn, &cs);
    out[2 * x] = cs * magnitude;
    out[2 * x + 1] = sn * magnitude;
  }
}

// For every token and each of `heads` heads: `width` channels at src + token * src_row + head *
// src_head go to dst (same indexing with the dst strides), the first 2 * half of them rotated.  src
// and dst may be the same memory: a thread takes a whole pair.
template <typename T>
__global__ void rotary_apply_kernel(const T* src, int src_row, int src_head, T* dst, int dst_row, int dst_head, int heads, int width,
                                    int half, int layout, const float* __restrict__ angles) {
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  const float* ang = angles + (size_t)tok * half * 2;
  const T* s = src + (size_t)tok * src_row;
  T* d = dst + (size_t)tok * dst_row;
  const int rest = width - 2 * half;                   // channels that pass
  const int per_head = half + rest;
  for (int x = threadIdx.x; x < heads * per_head; x += blockDim.x) {
    const int h = x / per_head, e = x % per_head;
    const T* sh = s + (size_t)h * src_head;
    T* dh = d + (size_t)h * dst_head;
    if (e < half) {
      const int iu = layout == ROTARY_INTERLEAVED ? 2 * e : e, iv = layout == ROTARY_INTERLEAVED ? 2 * e + 1 : e + half;
      const float u = to_f32(sh[iu]), v = to_f32(sh[iv]), cs = ang[2 * e], sn = ang[2 * e + 1];
      dh[iu] = from_f32<T>(fmaf(u, cs, -v * sn));
      dh[iv] = from_f32<T>(fmaf(v, cs, u * sn));
    } else if (src != dst || src_row != dst_row || src_head != dst_head) {
      dh[2 * half + e - half] = sh[2 * half + e - half];
    }
  }
}

Q25_EXPORT int q25_rotary_angles(const int* positions, const float* inv_freq, float magnitude, float* out, int n, int half, void* stream) {
  if (n <= 0 || half <= 0) return 0;
  const size_t total = (size_t)n * half;
  size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 8;
  if (blocks > most) blocks = most;
  launch(rotary_angles_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, positions, inv_freq, magnitude, out, n, half);
  return launch_status();
}

template <typename T>
static int rotary_apply(const void* src, int src_row, int src_head, void* dst, int dst_row, int dst_head, int n, int heads, int width,
                        int half, int layout, const float* angles, void* stream) {
  if (n <= 0 || heads <= 0) return 0;
  if (half < 0 || 2 * half > width || (layout != ROTARY_INTERLEAVED && layout != ROTARY_HALVES)) return (int)cudaErrorInvalidValue;
  const int work = heads * (width - half);
  launch(rotary_apply_kernel<T>, dim3(n), dim3(work >= 512 ? 256 : 128), 0, (cudaStream_t)stream, (const T*)src, src_row, src_head,
         (T*)dst, dst_row, dst_head, heads, width, half, layout, angles);
  return launch_status();
}
Q25_EXPORT int q25_rotary_apply_f32(const void* src, int sr, int sh, void* dst, int dr, int dh, int n, int heads, int width, int half,
                                    int layout, const float* angles, void* s) {
  return rotary_apply<float>(src, sr, sh, dst, dr, dh, n, heads, width, half, layout, angles, s);
}
Q25_EXPORT int q25_rotary_apply_bf16(const void* src, int sr, int sh, void* dst, int dr, int dh, int n, int heads, int width, int half,
                                     int layout, const float* angles, void* s) {
  return rotary_apply<bf16>(src, sr, sh, dst, dr, dh, n, heads, width, half, layout, angles, s);
}
