// Decode attention on tensor cores (bfloat16): the kernels for head sizes 16, 48, 80, ..., 240 (the kernel is in
// attention_mma.cuh, its entry points in attention_mma.cu).
#include "attention_mma.cuh"

namespace mll {

int launch_decode_mma_odd(const DecodeMmaArgs& a, int head_dim, int n_seqs, bool fused, cudaStream_t stream) {
  switch (head_dim) {
    case 16: return launch_decode_mma_sized<16>(a, n_seqs, fused, stream);
    case 48: return launch_decode_mma_sized<48>(a, n_seqs, fused, stream);
    case 80: return launch_decode_mma_sized<80>(a, n_seqs, fused, stream);
    case 112: return launch_decode_mma_sized<112>(a, n_seqs, fused, stream);
    case 144: return launch_decode_mma_sized<144>(a, n_seqs, fused, stream);
    case 176: return launch_decode_mma_sized<176>(a, n_seqs, fused, stream);
    case 208: return launch_decode_mma_sized<208>(a, n_seqs, fused, stream);
    case 240: return launch_decode_mma_sized<240>(a, n_seqs, fused, stream);
    default:
      mll_set_error("attention decode (mma): head_dim %d", head_dim);
      return -1;
  }
}

}  // namespace mll
