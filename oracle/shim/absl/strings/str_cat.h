// Test-infrastructure stand-in for abseil's str_cat.h (absent on this image); nothing from it is used.
#pragma once
