/* C-ML's include/nn/serving.h, served by libcml_b200: the scheduler is declared in cml_quant_api.h. */
#ifndef CML_B200_NN_SERVING_H
#define CML_B200_NN_SERVING_H
#include "../cml_quant_api.h"
#endif
