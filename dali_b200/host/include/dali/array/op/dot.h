// forwards to the op:: umbrella (reference: dali/array/op/dot.h)
#include "dali/array/op.h"
