// Defines the global the reference declares `extern` (interpolation.cpp:11); never dereferenced.
struct THCState;
THCState *state = nullptr;
