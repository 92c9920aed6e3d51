"""Browser chat UI for a finetuned model: ``create_server`` / ``serve``."""

from ohara_b200.webui.server import create_server, serve

__all__ = ["create_server", "serve"]
