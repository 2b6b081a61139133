/* C-ML's include/nn/paged_attention.h, served by libcml_b200: the paged KV cache and
 * cml_paged_gqa_forward are declared in cml_quant_api.h. */
#ifndef CML_B200_NN_PAGED_ATTENTION_H
#define CML_B200_NN_PAGED_ATTENTION_H
#include "../cml_quant_api.h"
#endif
