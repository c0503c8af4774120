// Image kernels of the embodied path (pure CUDA arithmetic, no graphics API):
//   resize_bilinear_u8   crop + bilinear resize of uint8 HWC images (the TF-style crop/resize the reference applies
//                        to camera frames before the VLA policy, siirl/engine/rollout/embodied_rollout.py:65-133)
//   raster_synth_env     observation renderer of the headless synthetic manipulation environment that stands in for
//                        LIBERO's MuJoCo off-screen camera: background gradient, goal disc, gripper disc with a
//                        shaded rim, written straight into a device buffer [N, H, W, 3] uint8
#include "common.cuh"
#include "launchers.h"

namespace sb {

__global__ void resize_bilinear_u8_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, int N,
                                          int H, int W, int C, int OH, int OW, float crop_y0, float crop_x0,
                                          float crop_h, float crop_w) {
  const long long total = (long long)N * OH * OW * C;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % C);
    const int ox = (int)((idx / C) % OW);
    const int oy = (int)((idx / ((long long)C * OW)) % OH);
    const int n = (int)(idx / ((long long)C * OW * OH));
    // pixel-centre sampling inside the crop window [crop_y0, crop_y0 + crop_h) x [crop_x0, crop_x0 + crop_w)
    const float sy = crop_y0 + (oy + 0.5f) * crop_h / OH - 0.5f;
    const float sx = crop_x0 + (ox + 0.5f) * crop_w / OW - 0.5f;
    const float fy = fminf(fmaxf(sy, 0.f), (float)(H - 1)), fx = fminf(fmaxf(sx, 0.f), (float)(W - 1));
    const int y0 = (int)floorf(fy), x0 = (int)floorf(fx);
    const int y1 = min(y0 + 1, H - 1), x1 = min(x0 + 1, W - 1);
    const float wy = fy - y0, wx = fx - x0;
    const unsigned char* im = src + (size_t)n * H * W * C;
    const float v00 = im[((size_t)y0 * W + x0) * C + c], v01 = im[((size_t)y0 * W + x1) * C + c];
    const float v10 = im[((size_t)y1 * W + x0) * C + c], v11 = im[((size_t)y1 * W + x1) * C + c];
    const float v = (1 - wy) * ((1 - wx) * v00 + wx * v01) + wy * ((1 - wx) * v10 + wx * v11);
    dst[idx] = (unsigned char)fminf(fmaxf(v + 0.5f, 0.f), 255.f);
  }
}

// state[n] = {agent_x, agent_y, goal_x, goal_y, gripper_open, _, _, _} in [0, 1] coordinates
__global__ void raster_synth_env_kernel(const float* __restrict__ state, unsigned char* __restrict__ out, int N, int H,
                                        int W) {
  const long long total = (long long)N * H * W;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(idx % W), y = (int)((idx / W) % H), n = (int)(idx / ((long long)W * H));
    const float* s = state + (size_t)n * 8;
    const float u = (x + 0.5f) / W, v = (y + 0.5f) / H;
    float r = 40.f + 60.f * v, g = 44.f + 50.f * u, b = 52.f + 30.f * (1.f - v);   // table-top gradient
    const float dg = sqrtf((u - s[2]) * (u - s[2]) + (v - s[3]) * (v - s[3]));
    if (dg < 0.06f) {
      r = 30.f; g = 200.f; b = 60.f;                                            // goal disc
    }
    const float da = sqrtf((u - s[0]) * (u - s[0]) + (v - s[1]) * (v - s[1]));
    const float rad = 0.035f + 0.015f * s[4];
    if (da < rad) {
      const float shade = 1.f - 0.5f * (da / rad) * (da / rad);               // shaded gripper disc
      r = 220.f * shade; g = 60.f * shade; b = 50.f * shade;
    }
    unsigned char* px = out + idx * 3;
    px[0] = (unsigned char)r; px[1] = (unsigned char)g; px[2] = (unsigned char)b;
  }
}

}  // namespace sb

using namespace sb;

static int img_grid(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = (long long)num_sms() * 8;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int sb_resize_bilinear_u8(const void* src, void* dst, int N, int H, int W, int C, int OH, int OW,
                                     float crop_y0, float crop_x0, float crop_h, float crop_w, cudaStream_t stream) {
  if (N == 0) return 0;
  resize_bilinear_u8_kernel<<<img_grid((long long)N * OH * OW * C), 256, 0, stream>>>(
      (const unsigned char*)src, (unsigned char*)dst, N, H, W, C, OH, OW, crop_y0, crop_x0, crop_h, crop_w);
  return (int)cudaGetLastError();
}

extern "C" int sb_raster_synth_env(const float* state, void* out, int N, int H, int W, cudaStream_t stream) {
  if (N == 0) return 0;
  raster_synth_env_kernel<<<img_grid((long long)N * H * W), 256, 0, stream>>>(state, (unsigned char*)out, N, H, W);
  return (int)cudaGetLastError();
}
