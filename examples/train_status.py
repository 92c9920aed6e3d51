"""Progress dashboard for a running training job, read straight from its log.

    python examples/train_status.py --log runs/speedrun.log --port 8082

The log has a line for every iteration, while experiment trackers only receive metrics on the
evaluation interval, so the loss curve here is dense and the time estimate follows the median step
time. Understands the multi-stage ``runs/speedrun.sh`` log (``[n/4] ...`` markers) as well as a
single pretraining or finetuning log; without ``--log`` the newest ``runs/*.log`` is used. The page
is self-contained (no external scripts or fonts), so it works on machines without internet access.
Same purpose and JSON fields as the reference dashboard (examples/train_status.py:45-170), with
wall-clock times reported in the machine's local timezone.
"""

from __future__ import annotations

import argparse
import json
import re
import statistics
from datetime import datetime, timedelta
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Any

_NUM = r"[\d.]+(?:e[+-]?\d+)?"
PATTERNS = {
    "step": re.compile(rf"^iter:\s*(?P<iter>\d+)\s*\|\s*loss:\s*(?P<loss>{_NUM})\s*\|\s*lr:\s*{_NUM}"
                       rf"\s*\|\s*time:\s*(?P<time>{_NUM})s"),
    "val": re.compile(rf"^iter:\s*(?P<iter>\d+)\s*\|\s*val_loss:\s*(?P<loss>{_NUM}).*?"
                      rf"val_acc:\s*(?P<acc>{_NUM})"),
    "stage": re.compile(r"^\[(?P<n>\d)/4\]\s*(?P<name>.+)$"),
    "budget": re.compile(r"budget:\s*[\d,]+\s*tokens over\s*(?P<iters>[\d,]+)\s*iters"),
    "horizon": re.compile(r"max_iters=(?P<iters>[\d,]+)"),
    "params": re.compile(r"params=(?P<n>[\d,]+)"),
}
_OPTIONAL = {"tokens_per_sec": re.compile(r"tok/s:\s*([\d,]+)"), "mfu": re.compile(r"mfu:\s*([\d.]+)%"),
             "eta": re.compile(r"eta:\s*([\d.]+)m"), "bpb": re.compile(r"val_bpb:\s*([\d.]+)")}


def _count(text: str) -> int:
    return int(text.replace(",", ""))


def _optional(name: str, line: str) -> float | None:
    hit = _OPTIONAL[name].search(line)
    return float(hit.group(1).replace(",", "")) if hit else None


def parse_log(path: Path, history_points: int = 300, total_override: int | None = None) -> dict[str, Any]:
    """Summarise a training log: stage, progress, pace, latest metrics and a thinned loss curve."""
    path = Path(path)
    now = datetime.now().astimezone()
    state: dict[str, Any] = {
        "stage": "waiting", "iter": 0, "total_iters": None, "loss": None,
        "median_step_seconds": None, "tokens_per_sec": None, "mfu": None, "params": None, "val": [],
        "history": [], "percent": 0.0, "remaining_minutes": None, "finish_at": None,
        "now": now.strftime("%H:%M"), "timezone": now.tzname(), "finished": False, "error": None,
        "log": str(path),
    }
    if not path.exists():
        state["error"] = f"log not found: {path}"
        return state

    curve: list[tuple[int, float]] = []
    step_times: list[float] = []
    declared_total = eta_minutes = None
    finetuning = False  # a single-file log has no stage markers; infer the stage from its lines
    with open(path, encoding="utf-8", errors="replace") as handle:
        for raw in handle:
            line = raw.rstrip("\n")
            if hit := PATTERNS["stage"].match(line):
                state["stage"] = hit["name"].strip()
                if hit["n"] == "4":  # finetuning restarts the iteration count
                    curve.clear()
                    declared_total = None
            elif "building SFT mixture" in line or "before SFT" in line:
                finetuning = True
            elif "after SFT" in line or "final val_loss" in line:
                state["finished"] = True
            elif hit := PATTERNS["budget"].search(line) or PATTERNS["horizon"].search(line):
                declared_total = _count(hit["iters"])
                if state["params"] is None and (p := PATTERNS["params"].search(line)):
                    state["params"] = _count(p["n"])
            elif (hit := PATTERNS["params"].search(line)) and state["params"] is None:
                state["params"] = _count(hit["n"])
            elif hit := PATTERNS["val"].match(line):
                state["val"].append({"iter": int(hit["iter"]), "loss": float(hit["loss"]),
                                     "acc": float(hit["acc"]), "bpb": _optional("bpb", line)})
            elif hit := PATTERNS["step"].match(line):
                state["iter"], state["loss"] = int(hit["iter"]), float(hit["loss"])
                step_times.append(float(hit["time"]))
                rate = _optional("tokens_per_sec", line)
                if rate is not None:
                    state["tokens_per_sec"] = int(rate)
                state["mfu"] = _optional("mfu", line)
                eta = _optional("eta", line)
                eta_minutes = eta if eta is not None else eta_minutes
                curve.append((state["iter"], state["loss"]))

    if state["stage"] == "waiting":
        state["stage"] = "supervised finetuning" if finetuning else "pretraining"
    # Step times are spiky; pace from the median of the most recent ones.
    median = statistics.median(step_times[-200:]) if step_times else None
    state["median_step_seconds"] = round(median, 3) if median else None
    total = total_override or declared_total
    if total is None and eta_minutes is not None and median:
        # eta is printed as (max_iters - iter) * mean step, so the horizon can be recovered from it.
        total = state["iter"] + round(eta_minutes * 60.0 / median)
    state["total_iters"] = total
    if total:
        state["percent"] = round(min(100.0, 100.0 * state["iter"] / total), 2)
        if median and not state["finished"]:
            remaining = max(0, total - state["iter"]) * median
            state["remaining_minutes"] = round(remaining / 60.0, 1)
            state["finish_at"] = (now + timedelta(seconds=remaining)).strftime("%H:%M")
    if state["finished"]:
        state["percent"], state["remaining_minutes"] = 100.0, 0.0
    stride = max(1, len(curve) // history_points)
    state["history"] = [{"i": i, "l": loss} for i, loss in curve[::stride]]
    return state


PAGE = """<!doctype html>
<html lang="en"><head><meta charset="utf-8">
<meta name="viewport" content="width=device-width, initial-scale=1">
<title>ohara_b200 training</title>
<style>
:root{color-scheme:light dark;--fg:#18181b;--bg:#fff;--dim:#71717a;--rail:#f4f4f5;--accent:#0d9488}
@media(prefers-color-scheme:dark){:root{--fg:#f4f4f5;--bg:#0b0b0c;--dim:#a1a1aa;--rail:#1f1f23}}
body{margin:0;background:var(--bg);color:var(--fg);font:15px/1.45 system-ui,sans-serif}
main{max-width:42rem;margin:0 auto;padding:2.5rem 1.5rem}
header{display:flex;gap:.75rem;align-items:center;margin-bottom:2rem}
header b{letter-spacing:-.01em} #stage{border:1px solid var(--rail);border-radius:99px;padding:.1rem .6rem;
font-size:12px;color:var(--dim)} #live{margin-left:auto;font-size:12px;color:var(--dim)}
#pct{font-size:4.5rem;font-weight:600;letter-spacing:-.04em;font-variant-numeric:tabular-nums}
.rail{height:10px;border-radius:99px;background:var(--rail);overflow:hidden;margin:.5rem 0}
#bar{height:100%;width:0;background:var(--accent);transition:width .8s}
.row{display:flex;justify-content:space-between;color:var(--dim);font-size:13px;margin-bottom:2.5rem}
.grid{display:grid;grid-template-columns:repeat(3,1fr);gap:1.5rem 2rem}
.k{font-size:11px;text-transform:uppercase;letter-spacing:.07em;color:var(--dim)}
.v{font-size:19px;font-variant-numeric:tabular-nums}
svg{width:100%;height:11rem;margin-top:.75rem} #note{margin-top:2.5rem;font-size:12px;color:var(--dim)}
</style></head><body><main>
<header><b>ohara_b200</b><span id="stage">-</span><span id="live"></span></header>
<div><span id="pct">-</span><span style="font-size:1.5rem;color:var(--dim)"> %</span></div>
<div class="rail"><div id="bar"></div></div>
<div class="row"><span id="iters">-</span><span id="eta"></span></div>
<div class="grid">
<div><div class="k">Train loss</div><div class="v" id="loss">-</div></div>
<div><div class="k">Val loss</div><div class="v" id="vloss">-</div></div>
<div><div class="k">Val bpb</div><div class="v" id="bpb">-</div></div>
<div><div class="k">Step</div><div class="v" id="step">-</div></div>
<div><div class="k">MFU</div><div class="v" id="mfu">-</div></div>
<div><div class="k">Tokens/s</div><div class="v" id="tps">-</div></div>
</div>
<div class="k" style="margin-top:2.75rem">Training loss <span id="npts"></span></div>
<svg viewBox="0 0 600 170" preserveAspectRatio="none"><path id="line" fill="none" stroke="#0d9488"
stroke-width="1.8" vector-effect="non-scaling-stroke"/></svg>
<div class="row" style="font-size:11px"><span id="lo"></span><span id="hi"></span></div>
<p id="note"></p></main>
<script>
const el = (id) => document.getElementById(id);
const fmt = (v, d) => (v === null || v === undefined ? "-" : Number(v).toFixed(d));
function path(points) {
  if (!points || points.length < 2) return {d: ""};
  const ys = points.map((p) => p.l), lo = Math.min(...ys), hi = Math.max(...ys), span = hi - lo || 1;
  const d = points.map((p, i) => (i ? "L" : "M") + (600 * i / (points.length - 1)).toFixed(1) + "," +
    (160 - 150 * (p.l - lo) / span).toFixed(1)).join(" ");
  return {d, lo, hi};
}
async function refresh() {
  try {
    const s = await (await fetch("/api/status", {cache: "no-store"})).json();
    el("pct").textContent = fmt(s.percent, 1);
    el("bar").style.width = s.percent + "%";
    el("stage").textContent = s.stage;
    el("iters").textContent = "iteration " + s.iter.toLocaleString() +
      (s.total_iters ? " of " + s.total_iters.toLocaleString() : "");
    el("eta").textContent = s.finished ? "finished" : !s.finish_at ? "" :
      (s.remaining_minutes > 90 ? (s.remaining_minutes / 60).toFixed(1) + " h" :
       Math.round(s.remaining_minutes) + " min") + " left, done ~" + s.finish_at + " " + s.timezone;
    el("loss").textContent = fmt(s.loss, 3);
    el("step").textContent = s.median_step_seconds ? fmt(s.median_step_seconds, 2) + "s" : "-";
    el("mfu").textContent = s.mfu === null ? "-" : fmt(s.mfu, 1) + "%";
    el("tps").textContent = s.tokens_per_sec ? s.tokens_per_sec.toLocaleString() : "-";
    const last = s.val.length ? s.val[s.val.length - 1] : null;
    el("vloss").textContent = last ? fmt(last.loss, 3) : "-";
    el("bpb").textContent = last && last.bpb !== null ? fmt(last.bpb, 4) : "-";
    const c = path(s.history);
    el("line").setAttribute("d", c.d);
    if (c.lo !== undefined) { el("lo").textContent = "min " + fmt(c.lo, 3); el("hi").textContent = "max " + fmt(c.hi, 3); }
    el("npts").textContent = s.history.length ? "(" + s.history.length + " points)" : "";
    el("live").textContent = s.finished ? "complete" : s.now + " " + s.timezone;
    el("note").textContent = s.error ? s.error :
      (s.params ? (s.params / 1e6).toFixed(0) + "M params, " : "") + "reading " + s.log;
  } catch (err) { el("live").textContent = "disconnected"; }
}
refresh(); setInterval(refresh, 4000);
</script></body></html>
"""


class StatusHandler(BaseHTTPRequestHandler):
    server_version = "ohara-b200-status"
    protocol_version = "HTTP/1.1"
    log_file: Path
    total_override: int | None = None

    def log_message(self, fmt: str, *args: Any) -> None:  # keep the terminal quiet
        return

    def _reply(self, body: bytes, content_type: str, status: int = 200) -> None:
        self.send_response(status)
        self.send_header("Content-Type", content_type)
        self.send_header("Cache-Control", "no-store")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_GET(self) -> None:  # noqa: N802 - name required by http.server
        route = self.path.split("?", 1)[0]
        if route in ("/", "/index.html"):
            self._reply(PAGE.encode(), "text/html; charset=utf-8")
        elif route == "/api/status":
            status = parse_log(self.log_file, total_override=self.total_override)
            self._reply(json.dumps(status).encode(), "application/json")
        else:
            self._reply(b'{"error":"not found"}', "application/json", 404)


def newest_log(directory: Path) -> Path | None:
    logs = sorted(directory.glob("*.log"), key=lambda p: p.stat().st_mtime)
    return logs[-1] if logs else None


def create_server(log: Path, host: str, port: int, total_iters: int | None = None) -> ThreadingHTTPServer:
    bound = type("BoundStatusHandler", (StatusHandler,), {"log_file": log, "total_override": total_iters})
    return ThreadingHTTPServer((host, port), bound)


def main() -> None:
    p = argparse.ArgumentParser(description="Serve a training progress dashboard")
    p.add_argument("--log", default=None, help="default: newest *.log under runs/")
    p.add_argument("--host", default="0.0.0.0")
    p.add_argument("--port", type=int, default=8082)
    p.add_argument("--total-iters", type=int, default=None,
                   help="pin the horizon for logs that do not print max_iters")
    args = p.parse_args()
    log = Path(args.log) if args.log else newest_log(Path("runs"))
    if log is None:
        raise SystemExit("no log files found in runs/; pass --log explicitly")
    print(f"reading {log}")
    server = create_server(log, args.host, args.port, args.total_iters)
    print(f"training status on http://{args.host}:{args.port}")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        print("\nshutting down")
    finally:
        server.shutdown()
        server.server_close()


if __name__ == "__main__":
    main()
