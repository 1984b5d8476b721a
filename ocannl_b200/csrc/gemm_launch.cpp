// placeholder until the contraction kernel lands
#include "runtime.hpp"
struct GemmLaunch {};
GemmLaunch* gemm_prepare(b200_routine*, int) { return nullptr; }
void gemm_enqueue(b200_routine*, int) {}
void gemm_release(GemmLaunch*) {}
