/* C-ML's include/nn/speculative.h, served by libcml_b200: the speculative decoder is declared in
 * cml_quant_api.h. */
#ifndef CML_B200_NN_SPECULATIVE_H
#define CML_B200_NN_SPECULATIVE_H
#include "../cml_quant_api.h"
#endif
