"""CUDA sources (sm_100a) and the code that compiles and loads them."""
