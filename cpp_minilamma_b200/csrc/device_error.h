// Error flags that device code raises instead of hanging or faulting: a bounded wait that ran out, a
// block whose shared memory is misplaced.  Each of the four kernels that can raise one keeps a flag of
// its own; this header names them for the code that brings them to the host.
#pragma once

// bit i of every mask below belongs to word[i]:
//   0 TMA linear kernel, 1 tcgen05 linear kernel, 2 tcgen05 prefill attention, 3 TMA decode attention
struct MllDeviceErrorWords {
  int* word[4];
};

// The current device's flag addresses (cached per device; the first call on a device must not come
// during a stream capture).  False when CUDA cannot give them; the words are then all null.
bool mll_device_error_words(MllDeviceErrorWords* words);
