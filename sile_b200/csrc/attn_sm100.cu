#include "internal.h"
namespace sile {
int attention_launch(const AttnProblem&, cudaStream_t) { return fail(SILE_ERR_UNSUPPORTED, "attention: not built yet"); }
}
