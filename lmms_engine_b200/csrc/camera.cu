// Pluecker camera-ray embedding for camera-controlled video generation: one thread per
// (view, pixel) builds the pixel-centre ray ((i+0.5-cx)/fx, (j+0.5-cy)/fy, 1), normalises it,
// rotates it by the camera-to-world rotation and writes [o x d, d] (6 floats), either in the
// [B,V,H,W,6] layout or directly channel-first [B,V,6,H,W] as the adapter's convolution wants.
// Reference: ray_condition, src/lmms_engine/models/wanvideo/wan_video_camera_controller.py:152-184
// (torch ops, on the CPU by default).
#include <cuda_runtime.h>

namespace b200 {

__global__ void plucker_kernel(const float* __restrict__ K, const float* __restrict__ c2w, float* __restrict__ out,
                               long views, int H, int W, int channels_first) {
  const long total = views * H * W;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long v = idx / (static_cast<long>(H) * W);
    const int pix = static_cast<int>(idx - v * H * W);
    const int j = pix / W, i = pix - j * W;
    const float* k = K + v * 4;
    const float* m = c2w + v * 16;
    float x = (i + 0.5f - k[2]) / k[0];
    float y = (j + 0.5f - k[3]) / k[1];
    float z = 1.f;
    const float inv = rsqrtf(x * x + y * y + z * z);
    x *= inv; y *= inv; z *= inv;
    const float dx = m[0] * x + m[1] * y + m[2] * z;
    const float dy = m[4] * x + m[5] * y + m[6] * z;
    const float dz = m[8] * x + m[9] * y + m[10] * z;
    const float ox = m[3], oy = m[7], oz = m[11];
    const float r[6] = {oy * dz - oz * dy, oz * dx - ox * dz, ox * dy - oy * dx, dx, dy, dz};
    if (channels_first) {
      float* o = out + v * 6 * H * W + pix;
#pragma unroll
      for (int c = 0; c < 6; ++c) o[static_cast<long>(c) * H * W] = r[c];
    } else {
      float* o = out + idx * 6;
#pragma unroll
      for (int c = 0; c < 6; ++c) o[c] = r[c];
    }
  }
}

}  // namespace b200

extern "C" int b200_plucker(const void* K, const void* c2w, void* out, long views, int H, int W, int channels_first,
                            cudaStream_t st) {
  const long total = views * H * W;
  if (total <= 0) return 0;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  b200::plucker_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      static_cast<const float*>(K), static_cast<const float*>(c2w), static_cast<float*>(out), views, H, W, channels_first);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
