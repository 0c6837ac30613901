// Device-timed probe of the C ABI without Python per-call overhead.
// usage: cprobe path dtype m n k ta tb [mode]   mode: 0 gemm, 1 affine fwd tanh, 2 bwd dX tanh,
//        3 bwd dW tanh, 4 bwd dW none
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <ginn_b200.h>

int main(int argc, char** argv) {
  if (argc < 8) return 2;
  int path = atoi(argv[1]), dtype = atoi(argv[2]);
  long m = atol(argv[3]), n = atol(argv[4]), k = atol(argv[5]);
  int ta = atoi(argv[6]), tb = atoi(argv[7]);
  int mode = argc > 8 ? atoi(argv[8]) : 0;
  size_t es = dtype == 0 ? 4 : 2;
  size_t big = (size_t)(m * k + k * n + 3 * m * n + m) * es;
  std::vector<char> h(big);
  for (size_t i = 0; i < big / es; ++i) {
    float v = ((int)(i * 2654435761u >> 20) % 200 - 100) / 400.f;
    if (dtype == 0) ((float*)h.data())[i] = v; else ((__half*)h.data())[i] = __float2half(v);
  }
  char* d;
  cudaMalloc(&d, big);
  cudaMemcpy(d, h.data(), big, cudaMemcpyHostToDevice);
  const int accum = getenv("ACC") ? 1 : 0;
  char *A = d, *B = A + m * k * es, *C = B + k * n * es, *Y = C + m * n * es, *dY = Y + m * n * es,
       *bias = dY + m * n * es;
  ginn_b200_set_option("force_path", path);
  auto run = [&]() -> int {
    if (mode == 0)
      return ginn_b200_gemm(0, nullptr, dtype, ta, tb, m, n, k, A, ta ? k : m, B, tb ? n : k, C, m, accum);
    if (mode == 1) {
      ginn_b200_pair p{A, m, B, k, k};
      return ginn_b200_affine_forward(0, nullptr, dtype, 1, &p, m, n, bias, 2, C, m);
    }
    ginn_b200_pair_grad g{A, m, B, k, k, nullptr, m, nullptr, k};
    if (mode == 2) g.db = B; else g.da = A;
    return ginn_b200_affine_backward(0, nullptr, dtype, 1, &g, m, n, dY, m, mode == 4 ? nullptr : Y, m,
                                     mode == 4 ? 0 : 2, nullptr);
  };
  for (int i = 0; i < (getenv("WARM") ? atoi(getenv("WARM")) : 3); ++i)
    if (int rc = run()) { printf("rc=%d %s\n", rc, ginn_b200_last_error()); return 1; }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int iters = getenv("ITERS") ? atoi(getenv("ITERS")) : 50;
  cudaEventRecord(e0);
  for (int i = 0; i < iters; ++i) run();
  cudaEventRecord(e1);
  cudaDeviceSynchronize();
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  double us = ms * 1000 / iters;
  printf("path %d dtype %d m%ld n%ld k%ld ta%d tb%d mode %d: %.1f us %.1f TFLOP/s status=%#x\n", path, dtype,
         m, n, k, ta, tb, mode, us, 2.0 * m * n * k / us / 1e6, ginn_b200_device_status(0, 1));
  return 0;
}
