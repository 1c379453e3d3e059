"""cpmcu: the reference's Python package layout (cpmcu/llm.py, cpmcu/speculative/*)
over libcpmcu_b200.so, a B200 (sm_100a) implementation of the speculative
decoding step.  `cpmcu.C` exposes the same functions as the reference's pybind
module of that name."""
