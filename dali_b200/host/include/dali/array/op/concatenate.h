// forwards to the op:: umbrella (reference: dali/array/op/concatenate.h)
#include "dali/array/op.h"
