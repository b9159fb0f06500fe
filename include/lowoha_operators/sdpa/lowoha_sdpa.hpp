// Same include path as in the reference tree (zendnnl/src/lowoha_operators/sdpa/lowoha_sdpa.hpp); the declarations live in
// zendnnl_b200/lowoha.hpp.
#pragma once
#include "zendnnl_b200/lowoha.hpp"
