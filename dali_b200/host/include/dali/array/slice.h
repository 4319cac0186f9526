// Slice, Broadcast and SlicingInProgress live in dali/array/array.h here (reference: dali/array/slice.h:13-60).
#include "dali/array/array.h"
