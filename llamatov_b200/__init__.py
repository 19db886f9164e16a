"""llamatov_b200: the Q8_0 transformer decode path as sm_100a CUDA behind the reference's
Python per-op interface (dev_residency / fact_dispatch names)."""
__version__ = "0.1"
