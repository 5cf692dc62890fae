"""The frozen HTTP contract of the control and inference API.

``openapi.json`` is the schema the application reports (``create_app(...).openapi()``), committed so that a change of a
route, a parameter or a response model shows up as a diff and fails ``tests/test_server_openapi.py`` until the file is
regenerated on purpose with ``python -m mfq_b200.server.protocol``.  WebSocket routes are not part of an OpenAPI schema;
:data:`WEBSOCKET_ROUTES` lists them.  Reference: ``mfq/server/protocol/openapi.json``.
"""

from __future__ import annotations

import json
from pathlib import Path

SCHEMA_PATH = Path(__file__).with_name("openapi.json")
WEBSOCKET_ROUTES = ("/api/v1/realtime",)


def current_schema() -> dict:
    from .. import ModelService, create_app
    return create_app(ModelService()).openapi()


def frozen_schema() -> dict:
    return json.loads(SCHEMA_PATH.read_text())


def write_schema() -> None:
    SCHEMA_PATH.write_text(json.dumps(current_schema(), indent=1, sort_keys=True) + "\n")
