// Host-side C shim over ferric_b200/csrc/layout.h so the CPU tests can drive the very index
// functions the device kernels use (compiled with g++, no CUDA needed).
#include "../../ferric_b200/csrc/layout.h"

extern "C" {
uint32_t shim_q4k_unit_offset(int r, int byte) { return ferric::q4k_unit_offset(r, byte); }
int shim_q4k_frag_weight(int s, int t, int j) { return ferric::q4k_frag_weight(s, t, j); }

uint32_t shim_q6k_unit_offset(int r, int byte) { return ferric::q6k_unit_offset(r, byte); }
int shim_q6k_frag_weight(int s, int t, int j) { return ferric::q6k_frag_weight(s, t, j); }

uint32_t shim_q5k_unit_offset(int r, int byte) { return ferric::q5k_unit_offset(r, byte); }
int shim_q5k_unit_bytes() { return ferric::kQ5KUnit; }
int shim_q4k_unit_bytes() { return ferric::kQ4KUnit; }
int shim_q6k_unit_bytes() { return ferric::kQ6KUnit; }
}
