"""Architecture families, one module each; importing this package registers them."""

from mlx_omnia_b200.architectures import muse_glimmer  # noqa: F401
