#pragma once
#include "utils/logging.hpp"
