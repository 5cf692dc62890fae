"""OpenAI/Anthropic-compatible inference server with control API and Prometheus metrics."""

from .app import create_app
from .service import ModelService

__all__ = ["create_app", "ModelService"]
