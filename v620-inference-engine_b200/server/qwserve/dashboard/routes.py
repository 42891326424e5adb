"""The dashboard's HTTP side.

``/`` and ``/dashboard`` serve the single page (read once, kept in memory, revalidated by ETag so that a browser
tab polling all day costs a 304); ``/metrics.json?tail=N`` serves the collector's payload with the newest N samples
of the history rings.  The page has no other assets: script and style are inline.
(The reference serves the same paths: server/qwserve/dashboard/routes.py:10-20.)"""
import hashlib
from pathlib import Path

from aiohttp import web

PAGE = Path(__file__).with_name("static") / "index.html"
DEFAULT_TAIL, MAX_TAIL = 300, 720          # samples of history sent to the page (5 s each: 25 min, one hour)


class DashboardRoutes:
    def __init__(self, collector):
        self.collector = collector
        self._body = PAGE.read_bytes()
        self._etag = '"' + hashlib.sha1(self._body).hexdigest()[:16] + '"'

    async def page(self, request: web.Request) -> web.Response:
        if request.headers.get("If-None-Match") == self._etag:
            return web.Response(status=304, headers={"ETag": self._etag})
        return web.Response(body=self._body, content_type="text/html", charset="utf-8", headers={"ETag": self._etag, "Cache-Control": "no-cache"})

    async def data(self, request: web.Request) -> web.Response:
        try:
            tail = int(request.query.get("tail", DEFAULT_TAIL))
        except ValueError:
            raise web.HTTPBadRequest(text="tail must be a number")
        return web.json_response(self.collector.payload(max(1, min(tail, MAX_TAIL))), headers={"Cache-Control": "no-store"})

    def table(self):
        return [web.get("/", self.page), web.get("/dashboard", self.page), web.get("/metrics.json", self.data)]


def add_routes(app: web.Application, collector) -> DashboardRoutes:
    routes = DashboardRoutes(collector)
    app.add_routes(routes.table())
    return routes
