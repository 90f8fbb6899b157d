// Test infrastructure: satisfies the one symbol the reference's offline module expects
// from its un-vendored grammar-compressor submodule, so that the reference's other graph
// preparation helpers can be compiled from their own sources and used as a checker.
#include <pybind11/pybind11.h>
void bind_batch_cpu(pybind11::module_&) {}
