// Host runtime of the native layer (data loading, checkpoint IO, schedules).
#pragma once
#include <stdint.h>
