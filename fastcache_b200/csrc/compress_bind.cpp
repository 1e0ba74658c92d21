#include <pybind11/pybind11.h>
void register_compress(pybind11::module_& m) {}
