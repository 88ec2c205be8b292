"""Seeded synthetic inputs for the tests: the generators live in ``proteusai_b200.synthetic`` (the benchmark uses
them too) and are re-exported here so that test code finds the data and the oracles side by side."""
from proteusai_b200.synthetic import STEP, chain_batch, draw_lengths, random_walk_chain, sigmas, wavenumbers  # noqa: F401
