// TEST INFRASTRUCTURE ONLY: empty stand-in; the CPU bodies use nothing from helper_cuda.h.
#pragma once
