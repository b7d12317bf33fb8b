/* Stand-in: everything lives in hip_runtime.h. Test infrastructure only. */
#include "hip_runtime.h"
