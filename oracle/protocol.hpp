// TEST INFRASTRUCTURE ONLY (CPU oracle; see fields.hpp).
#pragma once
#include "ops.hpp"
#include "hash.hpp"
