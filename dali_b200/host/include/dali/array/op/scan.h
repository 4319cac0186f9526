// forwards to the op:: umbrella (reference: dali/array/op/scan.h)
#include "dali/array/op.h"
