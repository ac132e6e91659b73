/* Compatibility shim: dnn.c callers include "norm.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_NORM_H
#define DNN_B200_SHIM_NORM_H
#include "dnn_b200.h"
#endif
