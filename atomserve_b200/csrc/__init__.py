"""CUDA sources (sm_100a) and the script that builds them into one shared library."""
