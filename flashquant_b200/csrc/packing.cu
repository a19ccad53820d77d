// 2-bit code packing: four codes per byte, first code in the top two bits.
// Byte-for-byte what pack_2bit / unpack_2bit of the reference's C++ core produce; pure
// streaming work: a thread turns 16 code bytes into 4 packed bytes (or back) with one
// 16-byte and one 4-byte access.
#include "fq_common.cuh"

namespace fq {

constexpr int kPackThreads = 256;

__global__ void __launch_bounds__(kPackThreads) pack_2bit_kernel(
    const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n_words,
    uint32_t* __restrict__ bad) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  uint32_t seen = 0;
  for (int64_t w = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; w < n_words; w += stride) {
    const uint4 c = reinterpret_cast<const uint4*>(codes)[w];
    const uint32_t in[4] = {c.x, c.y, c.z, c.w};
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bytes b0..b3 of the word hold codes 4i .. 4i+3
      const uint32_t v = in[i];
      seen |= v & 0xfcfcfcfcu;
      const uint32_t byte = ((v & 3u) << 6) | (((v >> 8) & 3u) << 4) | (((v >> 16) & 3u) << 2) |
                            ((v >> 24) & 3u);
      out |= byte << (8 * i);
    }
    reinterpret_cast<uint32_t*>(packed)[w] = out;
  }
  if (seen && bad) atomicOr(bad, 1u);
}

__global__ void __launch_bounds__(kPackThreads) unpack_2bit_kernel(
    const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes, int64_t n_words) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t w = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; w < n_words; w += stride) {
    const uint32_t p = reinterpret_cast<const uint32_t*>(packed)[w];
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t byte = (p >> (8 * i)) & 0xffu;
      out[i] = (byte >> 6) | (((byte >> 4) & 3u) << 8) | (((byte >> 2) & 3u) << 16) |
               ((byte & 3u) << 24);
    }
    reinterpret_cast<uint4*>(codes)[w] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

static int pack_grid(int64_t n_words) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (n_words + kPackThreads - 1) / kPackThreads;
  return int(want < int64_t(sms) * 8 ? want : int64_t(sms) * 8);
}

}  // namespace fq

using namespace fq;

extern "C" int fq_pack_2bit(const uint8_t* codes, uint8_t* packed, int64_t n_codes,
                            uint32_t* out_of_range, fq_stream_t stream) {
  FQ_RANGE("fq_pack_2bit");
  FQ_REQUIRE(n_codes >= 0 && n_codes % 16 == 0, FQ_ERR_INVALID_ARGUMENT,
             "fq_pack_2bit: %lld codes (a multiple of 16 is needed)", (long long)n_codes);
  if (n_codes == 0) return FQ_OK;
  FQ_REQUIRE(codes && packed, FQ_ERR_INVALID_ARGUMENT, "fq_pack_2bit: null pointer");
  FQ_REQUIRE(aligned(codes, 16) && aligned(packed, 4) && (!out_of_range || aligned(out_of_range, 4)),
             FQ_ERR_ALIGNMENT, "fq_pack_2bit: codes must be 16-byte and packed 4-byte aligned");
  const int64_t n_words = n_codes / 16;
  pack_2bit_kernel<<<pack_grid(n_words), kPackThreads, 0, stream>>>(codes, packed, n_words,
                                                                   out_of_range);
  return check_launch("pack_2bit kernel launch");
}

extern "C" int fq_unpack_2bit(const uint8_t* packed, uint8_t* codes, int64_t n_codes,
                              fq_stream_t stream) {
  FQ_RANGE("fq_unpack_2bit");
  FQ_REQUIRE(n_codes >= 0 && n_codes % 16 == 0, FQ_ERR_INVALID_ARGUMENT,
             "fq_unpack_2bit: %lld codes (a multiple of 16 is needed)", (long long)n_codes);
  if (n_codes == 0) return FQ_OK;
  FQ_REQUIRE(codes && packed, FQ_ERR_INVALID_ARGUMENT, "fq_unpack_2bit: null pointer");
  FQ_REQUIRE(aligned(codes, 16) && aligned(packed, 4), FQ_ERR_ALIGNMENT,
             "fq_unpack_2bit: codes must be 16-byte and packed 4-byte aligned");
  const int64_t n_words = n_codes / 16;
  unpack_2bit_kernel<<<pack_grid(n_words), kPackThreads, 0, stream>>>(packed, codes, n_words);
  return check_launch("unpack_2bit kernel launch");
}
