from .attention import AttentionMixer  # noqa: F401
from .mamba2 import Mamba2Mixer  # noqa: F401
from .latent_attention import LatentAttentionMixer  # noqa: F401
from .mingru import MinGRUMixer  # noqa: F401
from .delta import DeltaMixer  # noqa: F401
from .wkv import WKVMixer  # noqa: F401
