/* Compatibility shim: dnn.c callers include "nn.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_NN_H
#define DNN_B200_SHIM_NN_H
#include "dnn_b200.h"
#endif
