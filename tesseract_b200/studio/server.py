"""HTTP front of the visual-builder core (the reference's studio/app: a socket HTTP server with embedded assets).

    python -m tesseract_b200.studio.server --port 8765        # then open http://127.0.0.1:8765/

JSON API (request bodies are ``.tsb`` graphs unless noted):
  GET  /api/catalog                  the block palette
  POST /api/analyze                  diagnostics + inferred shapes
  POST /api/codegen?target=python|ir generated source  ->  {"source": ...}
  POST /api/import                   {"source": text}  ->  the graph embedded in a generated script
  POST /api/run                      runs the graph; the response is one JSON event per line, as they happen
  POST /api/cancel                   asks the running graph to stop
The page at ``/`` is a plain form over these calls (palette, graph text, analyze / generate / run buttons); the
node-canvas editor of the reference is a third-party browser library and is not bundled.
"""
from __future__ import annotations

import argparse
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

from .analysis import analyze
from .catalog import BlockCatalog
from .codegen import extract_tsb, generate_ir, generate_python
from .executor import Executor, RunOptions
from .graph import BlockGraph

_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>tesseract_b200 studio</title>
<style>body{font-family:sans-serif;margin:1.5em}textarea{width:100%;height:22em;font-family:monospace}
pre{background:#f4f4f4;padding:.6em;max-height:24em;overflow:auto}button{margin-right:.5em}</style></head><body>
<h2>tesseract_b200 studio</h2><p>Paste or edit a <code>.tsb</code> graph, then analyze, generate code or run it.
Block kinds: <span id="kinds"></span></p><textarea id="g"></textarea><p>
<button onclick="call('/api/analyze')">Analyze</button><button onclick="call('/api/codegen?target=python','source')">Python</button>
<button onclick="call('/api/codegen?target=ir','source')">IR</button><button onclick="run()">Run</button>
<button onclick="fetch('/api/cancel',{method:'POST'})">Cancel</button></p><pre id="out"></pre><script>
const out=document.getElementById('out'),g=document.getElementById('g');
fetch('/api/catalog').then(r=>r.json()).then(c=>{document.getElementById('kinds').textContent=c.map(b=>b.kind).join(', ')});
async function call(u,key){const r=await fetch(u,{method:'POST',body:g.value});const j=await r.json();
out.textContent=key&&j[key]?j[key]:JSON.stringify(j,null,2)}
async function run(){out.textContent='';const r=await fetch('/api/run',{method:'POST',body:g.value});
const rd=r.body.getReader(),d=new TextDecoder();for(;;){const{done,value}=await rd.read();if(done)break;
out.textContent+=d.decode(value);out.scrollTop=out.scrollHeight}}
</script></body></html>"""


class StudioServer(ThreadingHTTPServer):
    daemon_threads = True

    def __init__(self, addr, device: str = "cpu"):
        super().__init__(addr, _Handler)
        self.device = device
        self.cancel = threading.Event()
        self.run_lock = threading.Lock()


class _Handler(BaseHTTPRequestHandler):
    server: StudioServer
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt, *args):  # quiet by default
        pass

    def _send(self, code: int, body: bytes, ctype: str = "application/json") -> None:
        self.send_response(code)
        self.send_header("Content-Type", ctype)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def _json(self, obj, code: int = 200) -> None:
        self._send(code, json.dumps(obj).encode())

    def _body(self) -> str:
        n = int(self.headers.get("Content-Length", 0) or 0)
        return self.rfile.read(n).decode("utf-8") if n else ""

    def do_GET(self):
        path = urlparse(self.path).path
        if path == "/":
            self._send(200, _PAGE.encode(), "text/html; charset=utf-8")
        elif path == "/api/catalog":
            self._json(BlockCatalog.instance().to_json())
        else:
            self._json({"error": f"no such path '{path}'"}, 404)

    def do_POST(self):
        url = urlparse(self.path)
        text = self._body()
        try:
            if url.path == "/api/cancel":
                self.server.cancel.set()
                return self._json({"ok": True})
            if url.path == "/api/import":
                g = extract_tsb(json.loads(text).get("source", ""))
                return self._json(g.to_json() if g is not None else {"error": "no embedded graph found"}, 200 if g else 422)
            graph = BlockGraph.from_tsb(text)
            if url.path == "/api/analyze":
                return self._json(analyze(graph).to_json())
            if url.path == "/api/codegen":
                target = parse_qs(url.query).get("target", ["python"])[0]
                if target not in ("python", "ir"):
                    return self._json({"error": f"unknown target '{target}' (python | ir)"}, 400)
                return self._json({"source": generate_python(graph) if target == "python" else generate_ir(graph)})
            if url.path == "/api/run":
                return self._run(graph)
            self._json({"error": f"no such path '{url.path}'"}, 404)
        except (ValueError, KeyError, json.JSONDecodeError) as ex:
            self._json({"error": f"{type(ex).__name__}: {ex}"}, 400)

    def _run(self, graph: BlockGraph) -> None:
        if not self.server.run_lock.acquire(blocking=False):
            return self._json({"error": "a graph is already running"}, 409)
        try:
            self.server.cancel.clear()
            self.send_response(200)
            self.send_header("Content-Type", "application/x-ndjson")
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()

            def sink(ev):
                line = (json.dumps({"type": ev.type, "data": ev.data}) + "\n").encode()
                self.wfile.write(f"{len(line):x}\r\n".encode() + line + b"\r\n")
                self.wfile.flush()

            Executor.run(graph, sink, RunOptions(device=self.server.device, cancel=self.server.cancel))
            self.wfile.write(b"0\r\n\r\n")
        finally:
            self.server.run_lock.release()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8765)
    ap.add_argument("--device", default="cpu", help="cpu | cuda | cuda:N: where graphs run")
    a = ap.parse_args(argv)
    srv = StudioServer((a.host, a.port), a.device)
    print(f"studio: http://{a.host}:{srv.server_address[1]}/  (device {a.device})", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        srv.server_close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
