// The build of the persistent kernel with the hierarchical (cluster-first) grid barrier,
// launched in thread-block clusters when cluster_size is 2 or 4; see the note on build variants
// in mk_kernel.cu.
#define MK_VARIANT hier
#define MK_HIER_BARRIER 1
#define MK_VARIANT_SECONDARY 1
#include "mk_kernel.cu"
