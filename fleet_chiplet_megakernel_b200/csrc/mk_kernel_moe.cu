// The build of the persistent kernel that carries the mixture-of-experts ops (routing, per-expert
// row-owner linears, weighted combine); launched for graphs that hold them.  See the note on build
// variants in mk_kernel.cu.
#define MK_VARIANT moe
#define MK_WITH_MOE 1
#define MK_VARIANT_SECONDARY 1
#include "mk_kernel.cu"
