// forwards to the op:: umbrella (reference: dali/array/op/arange.h)
#include "dali/array/op.h"
