#pragma once
#include <ATen/cuda/Atomic.cuh>
