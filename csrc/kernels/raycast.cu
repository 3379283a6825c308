// Gate-race front camera as a CUDA ray caster: one thread per output pixel casts `samples` rays (one per shutter pose:
// motion blur) through a pinhole or an equidistant-fisheye lens at an analytic scene - a ground plane with a checker
// texture, yawed boxes (the bars of each gate, props) and upright cylinders (pillars) - shades the nearest hit with one
// sun and distance fog, and writes RGB into a headless device buffer [B, H, W, 3].
//
// Stands in for the reference's external OptiX renderer (src/dew/rl/hyperlux.py:90-260: per-drone scenes of gates,
// ground, sky, pillars, props; pinhole cameras resampled to a fisheye; a shutter's open and close cameras averaged).
#include <cuda_runtime.h>
#include <stdint.h>

namespace dewb {
namespace ray {

struct Hit { float t; float nx, ny, nz; float r, g, b; };

// box: center xyz, half extents xyz, yaw, rgb  (10 floats)
__device__ __forceinline__ void hit_box(const float* __restrict__ bx, float ox, float oy, float oz, float dx, float dy, float dz, Hit& h) {
  const float c = cosf(bx[6]), s = sinf(bx[6]);
  // ray in the box frame (rotate by -yaw about z)
  const float px = ox - bx[0], py = oy - bx[1], pz = oz - bx[2];
  const float lx = c * px + s * py, ly = -s * px + c * py, lz = pz;
  const float ex = c * dx + s * dy, ey = -s * dx + c * dy, ez = dz;
  float t0 = 0.f, t1 = h.t;
  int axis = -1; float sign = 0.f;
  const float lo[3] = {lx, ly, lz}, d[3] = {ex, ey, ez}, hf[3] = {bx[3], bx[4], bx[5]};
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    if (fabsf(d[a]) < 1e-12f) {
      if (fabsf(lo[a]) > hf[a]) return;
      continue;
    }
    const float inv = 1.f / d[a];
    float ta = (-hf[a] - lo[a]) * inv, tb = (hf[a] - lo[a]) * inv;
    float sg = -1.f;
    if (ta > tb) { const float tmp = ta; ta = tb; tb = tmp; sg = 1.f; }
    if (ta > t0) { t0 = ta; axis = a; sign = sg; }
    if (tb < t1) t1 = tb;
    if (t0 > t1) return;
  }
  if (axis < 0 || t0 <= 1e-4f || t0 >= h.t) return;
  float nx = 0.f, ny = 0.f, nz = 0.f;
  if (axis == 0) nx = sign; else if (axis == 1) ny = sign; else nz = sign;
  h.t = t0;
  h.nx = c * nx - s * ny; h.ny = s * nx + c * ny; h.nz = nz;
  h.r = bx[7]; h.g = bx[8]; h.b = bx[9];
}

// cylinder: center x, y, radius, height (from z = 0), rgb  (7 floats)
__device__ __forceinline__ void hit_cylinder(const float* __restrict__ cy, float ox, float oy, float oz, float dx, float dy, float dz, Hit& h) {
  const float px = ox - cy[0], py = oy - cy[1];
  const float a = dx * dx + dy * dy;
  if (a < 1e-12f) return;
  const float b = px * dx + py * dy;
  const float c = px * px + py * py - cy[2] * cy[2];
  const float disc = b * b - a * c;
  if (disc < 0.f) return;
  const float t = (-b - sqrtf(disc)) / a;
  if (t <= 1e-4f || t >= h.t) return;
  const float z = oz + t * dz;
  if (z < 0.f || z > cy[3]) return;
  const float inv = 1.f / cy[2];
  h.t = t;
  h.nx = (px + t * dx) * inv; h.ny = (py + t * dy) * inv; h.nz = 0.f;
  h.r = cy[4]; h.g = cy[5]; h.b = cy[6];
}

// cameras [B, samples, 12]: position xyz, then the rotation's columns: right, down, forward (world frame)
__global__ void raycast_kernel(const float* __restrict__ cameras, const float* __restrict__ boxes, const float* __restrict__ cylinders,
                               float* __restrict__ image, int B, int H, int W, int samples, int n_boxes, int n_cyl,
                               float tan_half, float half_fov, int fisheye, float fog, float checker) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(B) * H * W) return;
  const int x = static_cast<int>(idx % W), y = static_cast<int>((idx / W) % H), b = static_cast<int>(idx / (static_cast<long long>(W) * H));
  const float u = (x + 0.5f) / W * 2.f - 1.f, v = (y + 0.5f) / H * 2.f - 1.f;
  float cx, cyy, cz;       // ray in the camera frame (right, down, forward)
  bool held = true;
  if (fisheye) {
    const float rad = sqrtf(u * u + v * v);
    const float theta = half_fov * rad;
    held = theta < 1.5607963f;
    const float st = sinf(theta), ct = cosf(theta);
    const float k = rad > 1e-12f ? st / rad : 0.f;
    cx = u * k; cyy = v * k; cz = ct;
  } else {
    cx = u * tan_half; cyy = v * tan_half * (static_cast<float>(H) / W); cz = 1.f;
    const float inv = rsqrtf(cx * cx + cyy * cyy + cz * cz);
    cx *= inv; cyy *= inv; cz *= inv;
  }
  float acc_r = 0.f, acc_g = 0.f, acc_b = 0.f;
  const float sx = 0.3713907f, sy = 0.2785430f, sz = 0.8863914f;    // sun direction (normalised 0.4, 0.3, 0.955)
  for (int s = 0; s < samples && held; ++s) {
    const float* cam = cameras + (static_cast<long long>(b) * samples + s) * 12;
    const float ox = cam[0], oy = cam[1], oz = cam[2];
    const float dx = cam[3] * cx + cam[6] * cyy + cam[9] * cz;
    const float dy = cam[4] * cx + cam[7] * cyy + cam[10] * cz;
    const float dz = cam[5] * cx + cam[8] * cyy + cam[11] * cz;
    Hit h; h.t = 1e30f; h.nx = 0.f; h.ny = 0.f; h.nz = 1.f; h.r = 0.f; h.g = 0.f; h.b = 0.f;
    bool any = false;
    if (dz < -1e-6f && oz > 0.f) {                                   // ground plane z = 0, checker texture
      const float t = -oz / dz;
      h.t = t;
      const float gx = ox + t * dx, gy = oy + t * dy;
      const int cell = (static_cast<int>(floorf(gx / checker)) + static_cast<int>(floorf(gy / checker))) & 1;
      const float shade = cell ? 0.55f : 0.35f;
      h.r = shade * 0.9f; h.g = shade; h.b = shade * 0.8f;
      any = true;
    }
    const float t_before = h.t;
    for (int i = 0; i < n_boxes; ++i) hit_box(boxes + (static_cast<long long>(b) * n_boxes + i) * 10, ox, oy, oz, dx, dy, dz, h);
    for (int i = 0; i < n_cyl; ++i) hit_cylinder(cylinders + (static_cast<long long>(b) * n_cyl + i) * 7, ox, oy, oz, dx, dy, dz, h);
    any = any || h.t < t_before;
    // sky: a vertical gradient
    const float up = fminf(fmaxf(dz, 0.f), 1.f);
    const float sky_r = 0.65f - 0.35f * up, sky_g = 0.78f - 0.28f * up, sky_b = 0.95f - 0.10f * up;
    if (any) {
      const float lambert = fmaxf(h.nx * sx + h.ny * sy + h.nz * sz, 0.f);
      const float light = 0.35f + 0.65f * lambert;
      const float f = __expf(-fog * h.t);
      acc_r += f * h.r * light + (1.f - f) * sky_r;
      acc_g += f * h.g * light + (1.f - f) * sky_g;
      acc_b += f * h.b * light + (1.f - f) * sky_b;
    } else {
      acc_r += sky_r; acc_g += sky_g; acc_b += sky_b;
    }
  }
  const float inv = held ? 1.f / samples : 0.f;      // directions the lens does not hold are black
  float* out = image + idx * 3;
  out[0] = acc_r * inv; out[1] = acc_g * inv; out[2] = acc_b * inv;
}

}  // namespace ray
}  // namespace dewb

// cameras [B, samples, 12], boxes [B, n_boxes, 10], cylinders [B, n_cyl, 7], image [B, H, W, 3]; all fp32, contiguous.
extern "C" int dewb_raycast(const float* cameras, const float* boxes, const float* cylinders, float* image, int B, int H, int W,
                            int samples, int n_boxes, int n_cyl, float fov_degrees, int fisheye, float fog, float checker,
                            void* stream) {
  if (B <= 0 || H <= 0 || W <= 0 || samples <= 0 || checker <= 0.f) return -3;
  const float half = fov_degrees * 0.5f * 0.017453292519943295f;
  const long long n = static_cast<long long>(B) * H * W;
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  dewb::ray::raycast_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      cameras, boxes, cylinders, image, B, H, W, samples, n_boxes, n_cyl, tanf(half), half, fisheye, fog, checker);
  return static_cast<int>(cudaGetLastError());
}
