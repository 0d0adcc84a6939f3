// TEST INFRASTRUCTURE ONLY: the reference bodies include "var.h"; everything lives in op.h.
#pragma once
#include "op.h"
