from .model import Model  # noqa: F401
from . import falcon_h1  # noqa: F401  (registers FalconH1ForCausalLM)
from . import turevik  # noqa: F401  (registers Turevik)
from . import porarax  # noqa: F401  (registers Porarax)
from . import sogazen  # noqa: F401  (registers Sogazen)
from . import kimutar  # noqa: F401  (registers Kimutar)
