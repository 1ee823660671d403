// Test infrastructure (oracle build step), not product code.
// Force-included (-include) when compiling the reference's host sources with
// g++ 13: src/base/setup.h:96-116 defines print_vec (which streams xs[0]) before
// the operator<< template for vectors, so nested vectors fail two-phase lookup.
// Declaring the template first fixes that without touching the reference tree.
#pragma once
#include <iostream>
#include <vector>
template <typename T>
std::ostream& operator<<(std::ostream& out, std::vector<T> const& ts);
