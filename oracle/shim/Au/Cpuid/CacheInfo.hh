// Test-only stand-in: the reference includes this aocl-utils header but the files compiled for the
// cross-checks use nothing from it.
#pragma once
