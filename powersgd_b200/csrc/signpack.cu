// One-bit sign compression: pack, unpack, majority vote.
//
// Native replacement for the external `bit2byte` C++ extension that the research harness
// calls from its SignCompressor (paper-code/gradient_reducers.py:1206-1272): a flat float
// vector of `numel` entries, zero padded to a multiple of 32 and viewed as [32, L], becomes L
// int32 words; bit i of word l is 1 iff entry i*L + l is negative (zero and padding decode as
// +1, as in the original). One thread owns one word, so for every bit position the 32 lanes
// of a warp touch 32 consecutive floats: all traffic is coalesced and each thread keeps 32
// independent loads in flight.
#include "psgd_common.cuh"

constexpr int SIGN_THREADS = 256;

__global__ void __launch_bounds__(SIGN_THREADS) psgd_sign_pack_kernel(const float* __restrict__ src, long long numel,
                                                                        long long words, int* __restrict__ dst) {
  const long long l = (long long)blockIdx.x * SIGN_THREADS + threadIdx.x;
  if (l >= words) return;
  unsigned w = 0u;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const long long e = (long long)i * words + l;
    const float v = (e < numel) ? __ldg(src + e) : 0.f;
    w |= (v < 0.f ? 1u : 0u) << i;
  }
  dst[l] = (int)w;
}

__global__ void __launch_bounds__(SIGN_THREADS) psgd_sign_unpack_kernel(const int* __restrict__ src, long long numel,
                                                                          long long words, float scale,
                                                                          float* __restrict__ dst, int accumulate) {
  const long long l = (long long)blockIdx.x * SIGN_THREADS + threadIdx.x;
  if (l >= words) return;
  const unsigned w = (unsigned)src[l];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const long long e = (long long)i * words + l;
    if (e < numel) {
      const float s = ((w >> i) & 1u) ? -scale : scale;
      dst[e] = accumulate ? dst[e] + s : s;
    }
  }
}

// words_in: [voters, words]. mode 0: packed majority (ties decode as +1); mode 1: float
// sign(sum of +-1) in {-1, 0, +1} written to `dst_f`.
__global__ void __launch_bounds__(SIGN_THREADS) psgd_sign_vote_kernel(const int* __restrict__ words_in, int voters,
                                                                        long long numel, long long words, int mode,
                                                                        int* __restrict__ dst_w, float* __restrict__ dst_f) {
  const long long l = (long long)blockIdx.x * SIGN_THREADS + threadIdx.x;
  if (l >= words) return;
  unsigned out = 0u;
  for (int i = 0; i < 32; ++i) {
    int negatives = 0;
    for (int v = 0; v < voters; ++v) negatives += ((unsigned)__ldg(words_in + (long long)v * words + l) >> i) & 1u;
    const int sum = voters - 2 * negatives;  // sum of the +-1 votes
    if (mode == 0) {
      out |= (sum < 0 ? 1u : 0u) << i;
    } else {
      const long long e = (long long)i * words + l;
      if (e < numel) dst_f[e] = sum > 0 ? 1.f : (sum < 0 ? -1.f : 0.f);
    }
  }
  if (mode == 0) dst_w[l] = (int)out;
}

static inline int sign_blocks(long long words) { return (int)((words + SIGN_THREADS - 1) / SIGN_THREADS); }

PSGD_API int psgd_sign_pack(const float* src, long long numel, int* dst, cudaStream_t stream) {
  const long long words = (numel + 31) / 32;
  if (words == 0) return 0;
  psgd_sign_pack_kernel<<<sign_blocks(words), SIGN_THREADS, 0, stream>>>(src, numel, words, dst);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

PSGD_API int psgd_sign_unpack(const int* src, long long numel, float scale, float* dst, int accumulate,
                              cudaStream_t stream) {
  const long long words = (numel + 31) / 32;
  if (words == 0) return 0;
  psgd_sign_unpack_kernel<<<sign_blocks(words), SIGN_THREADS, 0, stream>>>(src, numel, words, scale, dst, accumulate);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

PSGD_API int psgd_sign_vote(const int* words_in, int voters, long long numel, int mode, int* dst_words, float* dst_float,
                            cudaStream_t stream) {
  const long long words = (numel + 31) / 32;
  if (words == 0) return 0;
  psgd_sign_vote_kernel<<<sign_blocks(words), SIGN_THREADS, 0, stream>>>(words_in, voters, numel, words, mode,
                                                                        dst_words, dst_float);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
