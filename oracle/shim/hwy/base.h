// Oracle build shim: the reference headers only need the name of Highway's
// half-precision storage type to declare templated (non-float) backends that
// the oracle never instantiates.
#pragma once
#include <cstdint>
namespace hwy
{
struct float16_t
{
  uint16_t bits;
};
} // namespace hwy
