// forwards to the op:: umbrella (reference: dali/array/op/binary.h)
#include "dali/array/op.h"
