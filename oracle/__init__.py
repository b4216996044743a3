"""CPU oracle for the Prioritized DCI hot path -- test infrastructure only.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this package.  The product (dciknn_cuda_b200) never does.
"""
