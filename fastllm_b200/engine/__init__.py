from .engine import LLMEngine  # noqa: F401
from .request import GenerationConfig, Request, RequestState  # noqa: F401
from .runner import EngineConfig, ModelRunner  # noqa: F401
