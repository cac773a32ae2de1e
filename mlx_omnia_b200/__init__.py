"""mlx_omnia_b200: a single-GPU (sm_100a) inference engine for the Muse-Glimmer decoder."""

__version__ = "0.1.0"
