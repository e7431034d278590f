// Peer-store bandwidth over NVLink against the number of thread blocks.
//
// Stand-alone microbenchmark (not part of the library) behind the thread-block limit of the pipelined
// transports: GPU 0 stores 512 MiB into GPU 1's memory (then, for comparison, into its own) in runs of
// 128 or 256 bytes that lie 512 KiB apart -- the pattern of a rotated store of the tile passes -- with
// 8-byte or 16-byte stores per lane, for grids of 8...296 blocks of 256 or 1024 threads.  Plain peer
// stores only: no bulk copies, no waits between kernels.  CUDA events around two launches after
// one warm-up launch.
//
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o peer_store_bandwidth benchmarks/peer_store_bandwidth.cu
//   ./peer_store_bandwidth            (needs two GPUs with peer access; prints one line per configuration)
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#define CK(x)                                                                   \
  do {                                                                          \
    cudaError_t e_ = (x);                                                       \
    if (e_ != cudaSuccess) {                                                    \
      std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
      std::exit(1);                                                             \
    }                                                                           \
  } while (0)

// Element e of the stream belongs to run e / runv; consecutive runs land stridev vectors apart
// (1024 runs per sweep of the destination), as the rows of a transposed tile do.
template <typename V>
__global__ void store_runs(V* dst, long long totalv, int runv, long long stridev) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < totalv; e += step) {
    const long long run = e / runv;
    const int within = (int)(e % runv);
    const long long off = (run % 1024) * stridev + (run / 1024) * runv + within;
    V v;
    memset(&v, 0, sizeof(V));
    dst[off] = v;
  }
}

int main() {
  int n = 0;
  CK(cudaGetDeviceCount(&n));
  if (n < 2) {
    std::printf("needs 2 GPUs\n");
    return 0;
  }
  int can = 0;
  CK(cudaDeviceCanAccessPeer(&can, 0, 1));
  if (!can) {
    std::printf("GPU 0 cannot access GPU 1\n");
    return 0;
  }
  CK(cudaSetDevice(0));
  CK(cudaDeviceEnablePeerAccess(1, 0));
  const long long bytes = 1LL << 29;
  void *local = nullptr, *remote = nullptr;
  CK(cudaMalloc(&local, bytes));
  CK(cudaSetDevice(1));
  CK(cudaMalloc(&remote, bytes));
  CK(cudaSetDevice(0));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (int target = 1; target >= 0; --target) {
    void* dst = target ? remote : local;
    for (int vb : {8, 16})
      for (int run_bytes : {128, 256})
        for (int threads : {256, 1024})
          for (int grid : {8, 16, 32, 48, 64, 96, 128, 148, 296}) {
            const long long totalv = bytes / vb;
            const int runv = run_bytes / vb;
            const long long stridev = totalv / 1024;
            auto launch = [&]() {
              if (vb == 8)
                store_runs<float2><<<grid, threads>>>((float2*)dst, totalv, runv, stridev);
              else
                store_runs<float4><<<grid, threads>>>((float4*)dst, totalv, runv, stridev);
            };
            launch();
            CK(cudaDeviceSynchronize());
            CK(cudaEventRecord(e0));
            launch();
            launch();
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float ms = 0.f;
            CK(cudaEventElapsedTime(&ms, e0, e1));
            ms /= 2;
            std::printf("%s vec=%2dB run=%3dB threads=%4d grid=%3d: %.3f ms %.0f GB/s\n", target ? "peer " : "local", vb,
                        run_bytes, threads, grid, ms, bytes / ms / 1e6);
          }
  }
  CK(cudaFree(local));
  CK(cudaSetDevice(1));
  CK(cudaFree(remote));
  return 0;
}
