// Shared between the term interpreter (generic.cu) and the kernel generator (rowgen.cu).
#pragma once
#include "../../include/tempest_b200.h"

namespace tb200 {
// Validates a group descriptor and works out, per phase, the bit mask of terms that phase evaluates
// (`need[p]`, p = 0..*phases, the last being the output sweep).  Returns a tb200_status.
int group_phases(const tb200_group_desc *d, unsigned long long *need, int *phases);
}  // namespace tb200
