// The fused dense-network kernel with ONE group of all 16 warps per CTA: for layers whose per-atom tensors are so large
// that two groups would each get a single atom, one group on a tile of two or more atoms shares every weight it
// fetches between the atoms and spreads an operation's units over twice the warps.
#define GB_FUSED_GROUPS 1
#include "chain_fused.cu"
