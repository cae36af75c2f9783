"""Multi-GPU: bootstrap, symmetric heap, tensor-parallel and particle-parallel paths."""
