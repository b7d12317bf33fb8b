#include <VX/vx.h>
