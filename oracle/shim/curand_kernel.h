// TEST INFRASTRUCTURE ONLY: stand-in so that sampleprocessing_op.cc (which includes <curand_kernel.h>
// even for its CPU body) compiles with a plain C++ compiler; the CPU body uses nothing from it.
#pragma once
