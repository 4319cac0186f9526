// forwards to the op:: umbrella (reference: dali/array/op/gather.h)
#include "dali/array/op.h"
