// C++ entry point of the engine.
// Replaces: src/include/fit_tsne.h:33-35 of the reference (same namespace and signature).
#ifndef TSNECUDA_B200_FIT_TSNE_H_
#define TSNECUDA_B200_FIT_TSNE_H_

#include "options.h"

namespace tsnecuda {

// Runs the whole pipeline (exact kNN, perplexity search, symmetrisation, FIt-SNE gradient loop) on
// opt.points and writes the embedding to opt.return_data (2*num_points floats, x block then y
// block).  Sets opt.trained and opt.trained_norm.  Invalid options print
// "E: Invalid options file. Terminating." and return, like the reference (src/fit_tsne.cu:38-42);
// other failures print "E: <reason>" and return with opt.trained == false (the reference exits the
// process).
void RunTsne(Options &opt, GpuOptions &gpu_opt);

}  // namespace tsnecuda
#endif
