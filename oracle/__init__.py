"""CPU oracle for the two hot paths (test infrastructure, not product code).

Everything in this package is a CPU restatement of the reference's PyTorch
formulation of the Wavefunction Embedding and the Geometric Attention.  It is
imported only by the tests, by the smoke check and by the CPU-baseline leg of
the benchmark.  The product path (the ``proteusai_b200`` package) never imports
it and has no CPU fallback.
"""
