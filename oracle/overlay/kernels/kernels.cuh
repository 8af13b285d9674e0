// Stand-in for the reference's src/kernels/kernels.cuh when its host is compiled against this library:
// the same namespace and the same eleven launcher signatures, forwarded to the C ABI of libredline_b200.so.
// (With this directory first on the include path the reference's `#include "kernels/kernels.cuh"`
// lands here; a maintainer of the reference would instead make src/kernels/kernels.cuh this one line.)
#include "../../../redline_llm_b200/csrc/kernels.cuh"
