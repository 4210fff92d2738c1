// Host build of the unit bit-gathering (tilus_b200/csrc/decode.cuh), used by
// tests/test_decode_host.py to check the kernels' extraction against the packer
// without a GPU.  Compiled with g++ by the test itself.
#include "decode.cuh"

using namespace b200q;

template <int VAR, int H>
static void fill(const uint32_t* w, uint32_t* raw, int* tgt) {
  raw[H] = pair_raw<VAR, H>(w);
  tgt[H] = pair_target<VAR, H>();
  if constexpr (H + 1 < 16) fill<VAR, H + 1>(w, raw, tgt);
}

template <int VAR>
static int dispatch(int var, const uint32_t* w, uint32_t* raw, int* tgt) {
  if (var == VAR) { fill<VAR, 0>(w, raw, tgt); return 0; }
  if constexpr (VAR + 1 < VAR_COUNT) return dispatch<VAR + 1>(var, w, raw, tgt);
  else return -1;
}

extern "C" int harness_unit_raw(int var, const uint32_t* words, uint32_t* raw16, int* target16) {
  return dispatch<0>(var, words, raw16, target16);
}
extern "C" int harness_var_bits(int var) { return var_bits(var); }
extern "C" int harness_var_bias(int var) { return var_bias(var); }
extern "C" int harness_var_count() { return VAR_COUNT; }
