// Bringing the kernels' error flags to the host.
//
// Two ways.  mll_take_device_error() copies the flags to the host and clears them; it synchronises
// with the device and is meant for callers that wait for their results anyway.  The sampling kernels
// (sampling.cu) read and clear the same flags on the device at the end of a step and pass them on in
// the status word that the host reads with the sampled tokens, so that a generation loop learns of a
// kernel that gave up without any copy or wait of its own.  mll_raise_device_error() sets flags from
// the host, for tests of the host's reaction: no kernel has to fail for them.
// The reference has no counterpart: its kernels have no waits that could run out.
#include "common.cuh"
#include "device_error.h"

extern "C" int* mll_linear_tma_error_address();
extern "C" int* mll_linear_tc5_error_address();
extern "C" int* mll_attn_tc5_error_address();
extern "C" int* mll_attn_decode_tma_error_address();

bool mll_device_error_words(MllDeviceErrorWords* words) {
  constexpr int kMaxDevices = 64;
  static MllDeviceErrorWords known[kMaxDevices];
  static bool have[kMaxDevices] = {false};
  for (int i = 0; i < 4; ++i) words->word[i] = nullptr;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return false;
  }
  if (!have[device]) {
    MllDeviceErrorWords found;
    found.word[0] = mll_linear_tma_error_address();
    found.word[1] = mll_linear_tc5_error_address();
    found.word[2] = mll_attn_tc5_error_address();
    found.word[3] = mll_attn_decode_tma_error_address();
    for (int i = 0; i < 4; ++i)
      if (found.word[i] == nullptr) return false;
    known[device] = found;
    have[device] = true;
  }
  *words = known[device];
  return true;
}

// The flags as a bit mask (see device_error.h), cleared; -1 if they cannot be read.  Synchronises.
MLL_API int mll_take_device_error() {
  MllDeviceErrorWords words;
  if (!mll_device_error_words(&words)) return -1;
  int mask = 0;
  const int zero = 0;
  for (int i = 0; i < 4; ++i) {
    int flag = 0;
    if (cudaMemcpy(&flag, words.word[i], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (flag) {
      if (cudaMemcpy(words.word[i], &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return -1;
      mask |= 1 << i;
    }
  }
  return mask;
}

// Sets the flags named in `mask` as a kernel that gave up would (for tests of the host side).
MLL_API int mll_raise_device_error(int mask) {
  MllDeviceErrorWords words;
  MLL_REQUIRE(mask >= 0 && mask < 16, "raise_device_error: mask %d names no flag", mask);
  MLL_REQUIRE(mll_device_error_words(&words), "raise_device_error: the flags' addresses cannot be had");
  const int one = 1;
  for (int i = 0; i < 4; ++i)
    if (mask & (1 << i))
      if (cudaMemcpy(words.word[i], &one, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return -2;
  return 0;
}
