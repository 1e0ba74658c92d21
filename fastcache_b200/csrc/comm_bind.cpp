#include <pybind11/pybind11.h>
void register_comm(pybind11::module_& m) {}
