// Call trace of one inference and the plan derived from it.
//
// A model compiled by Occamy is straight-line code: every inference issues the same
// runtime calls with the same shapes and the same pool offsets.  The runtime records the
// calls between cudnnCreate and cudnnDestroy (the compiled function's prologue and
// epilogue).  When an inference ends it looks for chains
//     convolution -> [+ bias [1,K,1,1]] -> [+ same-shape tensor] -> [ReLU | Clip]
// (and, for a few-channel stem convolution, a 3x3 / stride 2 max pool behind it)
// whose intermediate results nobody else reads before their memory is handed out again,
// and marks them.  The next time the same call sequence comes by, the convolution of such
// a chain is held back, the following calls are folded into its epilogue, and one kernel
// writes only the chain's final tensor.  A call that does not match the recorded sequence
// ends the speculation: whatever is held back is executed as it stands.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace occ {

enum Sym {
  S_POOLINIT = 1, S_MEMOFFSET, S_MALLOC, S_H2D, S_D2H, S_D2D, S_DEALLOC, S_POOLFREE,
  S_CONV, S_CONV_BIAS_ACT, S_TENSOR_OP, S_ACTIVE, S_CLIP, S_MAXPOOL, S_AVGPOOL, S_REDUCE,
  S_MATMUL, S_SOFTMAX, S_FLATTEN, S_RESHAPE, S_OPAQUE
};

enum Role { R_EAGER = 0, R_DEFER = 1, R_ABSORB = 2 };

// kind of a tensor-op / activation entry, as far as chains care
enum ChainKind {
  CK_NONE = 0, CK_BIAS_ADD = 1, CK_SAME_ADD = 2, CK_RELU = 3, CK_CLIP = 4,
  CK_POOL_3S2 = 5   // max pool 3x3, stride 2, pad 1
};

struct Entry {
  uint64_t sig = 1469598103934665603ull;
  int sym = 0;
  uintptr_t in[3] = {0, 0, 0};
  int64_t in_bytes[3] = {0, 0, 0};   // fp32 extent of each input (0: unknown, taken as one byte)
  uintptr_t out = 0;
  int64_t out_bytes = 0;   // fp32 extent of `out` (range size for the memory calls)
  int64_t dims[4] = {0, 0, 0, 0};
  int kind = CK_NONE;      // ChainKind, or the activation mode of a fused convolution
  bool fusable = false;    // convolution that the bf16 path takes (may head a chain)
  bool depthwise = false;
  bool poolable = false;   // convolution whose kernel can take a following CK_POOL_3S2 along
};

// Signature building.  Device pointers are taken relative to the active pool when they
// lie inside it; host pointers are left out of signatures.
Entry trace_entry(int sym);
void te_ptr(Entry &e, const void *p);
void te_i(Entry &e, int64_t v);
void te_f(Entry &e, float v);
void te_dims(Entry &e, const int64_t *d, int n);

// Records the call and returns the role the matching recorded program gives it.
// *deviated is set when this call is the first of the inference that matches no recorded
// program although earlier calls did.
Role trace_step(Entry &e, bool *deviated);

void trace_begin();                 // cudnnCreate
void trace_end();                   // cudnnDestroy: analyse and store if the sequence is new
void trace_set_pool(void *base, size_t bytes);
void trace_note_elided();           // a tensor of this inference was skipped by a fusion
bool trace_has_elided();
bool trace_enabled();
void trace_set_enabled(bool on);   // turning it off also forgets the recorded programs
int64_t trace_fused_chains();       // chains executed fused since load
void trace_count_chain();

}  // namespace occ
