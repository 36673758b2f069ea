// The tensor-parallel build of the persistent kernel: the same source with the exchange code
// compiled in (linear epilogues that push their sums to every rank, input staging that gathers
// them).  Launched whenever world_size > 1; see the note on build variants in mk_kernel.cu.
#define MK_VARIANT tp
#define MK_WITH_XCHG 1
#define MK_VARIANT_SECONDARY 1
#include "mk_kernel.cu"
