/* Compatibility shim: dnn.c callers include "ops.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_OPS_H
#define DNN_B200_SHIM_OPS_H
#include "dnn_b200.h"
#endif
