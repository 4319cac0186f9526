// forwards to the op:: umbrella (reference: dali/array/op/reducers.h)
#include "dali/array/op.h"
