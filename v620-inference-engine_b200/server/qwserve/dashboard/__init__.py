"""Built-in dashboard: a one-page view of throughput, queue, prefix-cache and GPU telemetry, fed by
``/metrics.json`` (reference behaviour: server/qwserve/dashboard/__init__.py:7-15)."""
from .collector import Collector
from .metrics import Metrics
from .routes import add_routes


def attach(app, server):
    col = Collector(server)
    add_routes(app, col)

    async def start(_app):
        col.start()

    async def stop(_app):
        col.stop()
    app.on_startup.append(start)
    app.on_cleanup.append(stop)
    return col
