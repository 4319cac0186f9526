// forwards to the op:: umbrella (reference: dali/array/op/reducer_operation.h)
#include "dali/array/op.h"
