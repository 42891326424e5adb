"""HTTP routes of the dashboard: the page at ``/`` and ``/dashboard``, its data at ``/metrics.json``."""
import os

from aiohttp import web

STATIC = os.path.join(os.path.dirname(__file__), "static")


def add_routes(app, collector):
    async def index(_):
        return web.FileResponse(os.path.join(STATIC, "index.html"))

    async def metrics(request):
        return web.json_response(collector.payload(int(request.query.get("tail", 300))))
    app.router.add_get("/", index)
    app.router.add_get("/dashboard", index)
    app.router.add_get("/metrics.json", metrics)
