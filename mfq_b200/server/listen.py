"""Listeners: one application served on several ports (an OpenAI-facing and an Anthropic-facing one by default).

Both ports serve every route; two ports exist so that clients configured with only a base URL and a vendor SDK can be
pointed at "their" port, as with the reference (``mfq serve``: 8090 OpenAI, 8091 Anthropic,
``mfq/commands/serve.py:271-437``).  Each listener is a ``uvicorn.Server`` in its own thread; ``stop()`` asks all of
them to exit and joins the threads.
"""

from __future__ import annotations

import threading
import time


class Listeners:
    def __init__(self, app, host: str, ports: list[int], access_log: bool = False) -> None:
        import uvicorn
        self.servers = [uvicorn.Server(uvicorn.Config(app, host=host, port=p, access_log=access_log, log_level="warning"))
                        for p in dict.fromkeys(ports)]
        self.threads: list[threading.Thread] = []

    def start(self, wait: float = 10.0) -> "Listeners":
        for s in self.servers:
            s.install_signal_handlers = lambda: None  # threads other than the main one cannot install handlers
            t = threading.Thread(target=s.run, daemon=True)
            t.start()
            self.threads.append(t)
        end = time.time() + wait
        while time.time() < end and not all(s.started for s in self.servers):
            time.sleep(0.02)
        if not all(s.started for s in self.servers):
            self.stop()
            raise RuntimeError("a listener did not come up (port in use?)")
        return self

    def ports(self) -> list[int]:
        return [sock.getsockname()[1] for s in self.servers for srv in s.servers for sock in srv.sockets]

    def stop(self) -> None:
        for s in self.servers:
            s.should_exit = True
        for t in self.threads:
            t.join(timeout=10)

    def wait(self) -> None:
        try:
            while any(t.is_alive() for t in self.threads):
                time.sleep(0.2)
        except KeyboardInterrupt:
            self.stop()
