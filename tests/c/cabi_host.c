/* A host program in plain C that uses the library through its C ABI only: device buffers from the CUDA
 * runtime, no Python, no torch.  INT8 per-tensor fake quantisation of a small fp32 vector, checked
 * against the same arithmetic done on the host; then the argument validation (status codes). */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "b200q.h"

#define N 4096

int main(void) {
  float *hx = (float*)malloc(N * sizeof(float)), *hy = (float*)malloc(N * sizeof(float));
  float hmax = 0.f;
  for (int i = 0; i < N; ++i) {
    hx[i] = sinf(0.37f * (float)i) * (1.f + (float)(i % 7));
    if (fabsf(hx[i]) > hmax) hmax = fabsf(hx[i]);
  }
  float *dx, *dy, *damax;
  if (cudaMalloc((void**)&dx, N * sizeof(float)) || cudaMalloc((void**)&dy, N * sizeof(float)) ||
      cudaMalloc((void**)&damax, sizeof(float))) return 2;
  cudaMemcpy(dx, hx, N * sizeof(float), cudaMemcpyHostToDevice);
  cudaMemset(damax, 0, sizeof(float));
  int st = b200q_amax_tensor(dx, N, B200Q_F32, damax, NULL);
  if (st != B200Q_OK) { printf("amax: %s\n", b200q_strerror(st)); return 3; }
  st = b200q_fake_int_tensor(dx, dy, N, B200Q_F32, damax, 8, 0, 1, NULL);
  if (st != B200Q_OK) { printf("fake_int: %s\n", b200q_strerror(st)); return 4; }
  float amax;
  cudaMemcpy(&amax, damax, sizeof(float), cudaMemcpyDeviceToHost);
  cudaMemcpy(hy, dy, N * sizeof(float), cudaMemcpyDeviceToHost);
  if (cudaDeviceSynchronize() != cudaSuccess) return 5;
  if (amax != hmax) { printf("amax %g != %g\n", amax, hmax); return 6; }
  const float scale = 127.f / amax;
  for (int i = 0; i < N; ++i) {
    float r = rintf(hx[i] * scale);
    r = r > 127.f ? 127.f : (r < -127.f ? -127.f : r);
    const float want = r / scale;
    if (hy[i] != want) { printf("element %d: %g != %g\n", i, hy[i], want); return 7; }
  }
  if (b200q_fake_int_tensor(NULL, dy, N, B200Q_F32, damax, 8, 0, 1, NULL) != B200Q_ERR_NULL) return 8;
  if (b200q_fake_int_tensor(dx, dy, N, 99, damax, 8, 0, 1, NULL) != B200Q_ERR_DTYPE) return 9;
  if (b200q_fake_int_tensor(dx + 1, dy, N - 1, B200Q_F32, damax, 8, 0, 1, NULL) != B200Q_ERR_ALIGN) return 10;
  printf("cabi_host ok: version %d, %d SMs\n", b200q_version(), b200q_sm_count());
  return 0;
}
