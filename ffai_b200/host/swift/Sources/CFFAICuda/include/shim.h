/* Umbrella header of the CFFAICuda module: the C ABI of libffai_cuda, nothing else.
 * Build with -Xcc -I<repo>/include so that the header below resolves. */
#include "ffai_cuda.h"
