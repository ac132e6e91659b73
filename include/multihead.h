/* Compatibility shim: dnn.c callers include "multihead.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_MULTIHEAD_H
#define DNN_B200_SHIM_MULTIHEAD_H
#include "dnn_b200.h"
#endif
