// Micro-benchmark of the key walk's inner loop (walk_quant.cuh: quant_upper4 / quant_bottom4,
// the four-column PTX walk of a group of 8 levels) with everything else of the kernels taken
// away: one block per SM, node pieces and a key tile of F = 2000 in shared memory filled with
// random but valid contents, W warps walking the same group over and over (each round starts
// at an address that depends on the previous result, so nothing can be hoisted).  Prints clocks
// per warp-step (one level of one column for 32 rows) per scheduler -- the rate the walk
// kernels could reach if staging, hand-offs and leaf sums cost nothing.
//
//   make -C treebeard_b200/csrc probes && treebeard_b200/lib/walk_step_probe [rounds]
#include "../walk_quant.cuh"

#include <cstdio>
#include <cstdlib>

using namespace tb;

constexpr int kKeyBytes = quant_key_tile_bytes(2000);

__global__ void __launch_bounds__(768, 1) walk_step_probe(uint32_t *out, unsigned long long *cyc, int rounds, int warps_active,
                                                          uint32_t zero) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t *ring = reinterpret_cast<uint32_t *>(smem); // upper-level piece, bottom-level piece
  uint16_t *keys = reinterpret_cast<uint16_t *>(smem + 2 * kQPiece);
  uint32_t h = 12345u + tid * 2654435761u + blockIdx.x;
  for (int i = tid; i < 2 * kQPiece / 4; i += blockDim.x) {
    h = h * 1664525u + 1013904223u + i;
    const uint32_t f = (h >> 8) % 2000u, code = (f >> 1) * 64u + (f & 1u), key = 1024u + (h >> 3) % 30720u;
    ring[i] = (code << 16) | key;
  }
  for (int i = tid; i < kKeyBytes / 2; i += blockDim.x) {
    h = h * 1664525u + 1013904223u + i;
    keys[i] = (uint16_t)(1024u + (h >> 5) % 30720u);
  }
  __syncthreads();
  if (warp >= warps_active) return;
  const uint32_t ring_s = smem_u32(ring), keys_lane = smem_u32(keys) + lane * 4u;
  const int sw = warp & 7;
  uint32_t colb[4];
  for (int c = 0; c < 4; ++c) colb[c] = ring_s + (((uint32_t)(lane + sw + 8 * c) & 31u) * 4u);
  uint32_t acc = 0, ties = 0;
  const long long t0 = clock64();
#pragma unroll 1
  for (int r = 0; r < rounds; ++r) {
    uint32_t A[4], bot[4], cu[4], cx[4];
    for (int c = 0; c < 4; ++c) {
      A[c] = colb[c] + (acc & zero);
      bot[c] = A[c] + kQPiece;
      cu[c] = 128u - A[c];
      cx[c] = cu[c] + bot[c] - A[c] - 128u * 127u;
    }
    quant_upper4<8>(A, ties, keys_lane, cu, cx);
    quant_bottom4(A, ties, keys_lane, bot);
    acc += A[0] + A[1] + A[2] + A[3];
  }
  const long long t1 = clock64();
  if (lane == 0 && warp == 0) cyc[blockIdx.x] = (unsigned long long)(t1 - t0);
  out[blockIdx.x * blockDim.x + tid] = acc + ties;
}

int main(int argc, char **argv) {
  const int rounds = argc > 1 ? atoi(argv[1]) : 2000;
  cudaDeviceProp pr;
  if (cudaGetDeviceProperties(&pr, 0) != cudaSuccess) {
    printf("no CUDA device\n");
    return 1;
  }
  const int sms = pr.multiProcessorCount;
  uint32_t *out;
  unsigned long long *cyc;
  cudaMalloc(&out, (size_t)sms * 768 * 4);
  cudaMalloc(&cyc, (size_t)sms * 8);
  const int smem = 2 * kQPiece + kKeyBytes;
  cudaFuncSetAttribute(walk_step_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int warps : {4, 8, 16, 24}) {
    for (int w = 0; w < 2; ++w) {
      walk_step_probe<<<sms, 768, smem>>>(out, cyc, rounds, warps, 0u);
      const cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) {
        printf("error: %s\n", cudaGetErrorString(e));
        return 1;
      }
    }
    unsigned long long c0 = 0;
    cudaMemcpy(&c0, cyc, 8, cudaMemcpyDeviceToHost);
    const double steps = (double)rounds * 32.0 * warps; // 4 columns x 8 levels per round and warp
    printf("%2d warps per SM: %7.1f clocks per round, %5.2f clocks per warp-step per scheduler\n", warps, (double)c0 / rounds,
           (double)c0 / steps * 4.0);
  }
  return 0;
}
