"""The parts a layer is put together from.  Importing this package registers them."""
from . import attention, block, embedding, feedforward, latent_attention, moe, norm, rope, wkv  # noqa: F401
