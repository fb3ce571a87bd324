"""TEST INFRASTRUCTURE ONLY.  CPU restatements of the reference's tree-attention decode used
to check the CUDA path.  Nothing in the product imports this package: only tests/,
__graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs do, and only as
the checker or as the timed CPU baseline."""
