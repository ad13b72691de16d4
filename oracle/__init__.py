"""TEST INFRASTRUCTURE ONLY -- the checkers of the CUDA path, never part of it.

  neighbors_oracle.py  numpy restatement of the reference's neighbour searches, keep rule, cutoffs (fixed and adaptive)
  pet_oracle.py        torch-CPU restatement of the network and of the force/virial folds
  reference_lib.py     ctypes access to the reference's own sources compiled for the host (build_ref.sh, ref_driver.cpp,
                       kokkos_host/): what the two restatements and the CUDA path are held to

Only tests/, __graft_entry__.smoke() and bench.py's CPU arms import this package; nothing under pet_kokkos_b200/ does
(tests/test_library.py checks it).
"""
