// forwards to the op:: umbrella (reference: dali/array/op/eye.h)
#include "dali/array/op.h"
