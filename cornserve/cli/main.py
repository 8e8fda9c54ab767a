"""``cornserve`` command-line client (reference: python/cornserve/cli/main.py:148-889).

  cornserve up [--num-gpus N] [--cpu]          start the local control plane (the counterpart of applying the
                                               Kubernetes manifests): resource manager + sidecars, task dispatcher,
                                               gateway, as processes of this machine
  cornserve register app.py [--alias NAME]     deploy an app; streams progress and executor logs
  cornserve unregister APP                     APP is an app id or an alias
  cornserve list
  cornserve invoke APP DATA [--aggregate-keys choices.0.delta.content] [--png-key KEY --save-png-path F]
                            [--audio-key KEY --save-audio-path F]
                                               DATA is JSON / YAML text, a file path, or - for stdin
  cornserve tasklib deploy PACKAGE_OR_DIR | purge
  cornserve deploy_profiles DIR [--dry-run]
  cornserve scale TASK_ID NUM_GPUS
"""

from __future__ import annotations

import argparse
import base64
import json
import os
import sys
from pathlib import Path
from typing import Any

import requests
import yaml

from ..constants import GATEWAY_URL, STATE_DIR
from .audio_streamer import PCMStreamPlayer
from .log_streamer import LogStreamer


def gateway_url() -> str:
    return os.environ.get("CORNSERVE_GATEWAY_URL", GATEWAY_URL).rstrip("/")


class Alias:
    """``alias -> app id`` kept in ``<state dir>/alias.json``."""

    def __init__(self, path: Path | None = None) -> None:
        self.path = path or Path(STATE_DIR) / "alias.json"
        self.map: dict[str, str] = json.loads(self.path.read_text()) if self.path.exists() else {}

    def _save(self) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.path.write_text(json.dumps(self.map, indent=1))

    def get(self, alias: str) -> str | None:
        return self.map.get(alias)

    def reverse_get(self, app_id: str) -> str | None:
        return next((a for a, i in self.map.items() if i == app_id), None)

    def set(self, app_id: str, alias: str) -> None:
        if alias.startswith("app-"):
            raise ValueError("aliases may not start with 'app-' (reserved for app ids)")
        self.map[alias] = app_id
        self._save()

    def remove(self, alias_or_id: str) -> None:
        for a in [a for a, i in self.map.items() if a == alias_or_id or i == alias_or_id]:
            del self.map[a]
        self._save()

    def resolve(self, name: str) -> str:
        return self.map.get(name, name)


def load_payload(arg: str) -> dict[str, Any]:
    """JSON or YAML given literally, as a file path, or on stdin (``-``)."""
    if arg == "-":
        text = sys.stdin.read()
    elif os.path.exists(arg):
        text = Path(arg).read_text()
    else:
        text = arg
    try:
        data = json.loads(text)
    except json.JSONDecodeError:
        data = yaml.safe_load(text)
    if not isinstance(data, dict):
        raise ValueError("the request payload must be a mapping")
    return data


def extract_nested(data: Any, dotted: str) -> Any:
    """``choices.0.delta.content`` style lookup; missing parts yield ``None``."""
    cur = data
    for part in dotted.split("."):
        if isinstance(cur, list):
            try:
                cur = cur[int(part)]
            except (ValueError, IndexError):
                return None
        elif isinstance(cur, dict):
            cur = cur.get(part)
        else:
            return None
        if cur is None:
            return None
    return cur


def save_png(b64: str, path: str | None) -> str:
    data = base64.b64decode(b64)
    if data[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("the selected field does not hold a PNG image")
    out = path or "cornserve_output.png"
    Path(out).write_bytes(data)
    return out


# ------------------------------------------------------------------------------------------------------
# commands
# ------------------------------------------------------------------------------------------------------
def cmd_register(a: argparse.Namespace) -> int:
    src = Path(a.path).read_text()
    alias = a.alias or Path(a.path).stem
    streamer = None
    try:
        with requests.post(f"{gateway_url()}/app/register", json={"source_code": src}, stream=True, timeout=3600) as r:
            if r.status_code != 200:
                print(f"registration failed: {r.status_code} {r.text}", file=sys.stderr)
                return 1
            app_id = None
            for line in r.iter_lines():
                if not line or not line.startswith(b"data: "):
                    continue
                ev = json.loads(line[6:])["event"]
                if ev["type"] == "initial":
                    app_id = ev["app_id"]
                    Alias().set(app_id, alias)
                    print(f"app {app_id} (alias {alias}): deploying {len(ev['task_names'])} unit tasks: {', '.join(ev['task_names'])}")
                    if not a.no_logs:
                        streamer = LogStreamer(ev["task_names"]).start()
                elif ev["type"] == "final":
                    print(ev["message"])
                    print(f"invoke with: cornserve invoke {alias} '<json>'")
                    return 0
                else:
                    print(f"registration failed: {ev['message']}", file=sys.stderr)
                    if app_id:
                        Alias().remove(app_id)
                    return 1
        return 1
    finally:
        if streamer is not None:
            streamer.stop()


def cmd_unregister(a: argparse.Namespace) -> int:
    al = Alias()
    app_id = al.resolve(a.app)
    r = requests.post(f"{gateway_url()}/app/unregister/{app_id}", timeout=600)
    if r.status_code == 404:
        print(f"app {app_id} not found", file=sys.stderr)
        return 1
    r.raise_for_status()
    al.remove(app_id)
    print(f"app {app_id} unregistered")
    return 0


def cmd_list(a: argparse.Namespace) -> int:
    r = requests.get(f"{gateway_url()}/app/list", timeout=30)
    r.raise_for_status()
    al = Alias()
    apps = r.json()
    if not apps:
        print("no apps registered")
    for app_id, status in apps.items():
        print(f"{app_id:40s} {al.reverse_get(app_id) or '-':20s} {status}")
    return 0


def cmd_invoke(a: argparse.Namespace) -> int:
    app_id = Alias().resolve(a.app)
    payload = load_payload(a.data)
    player = PCMStreamPlayer(sample_rate=a.sample_rate, play=not a.no_play) if a.audio_key else None
    with requests.post(f"{gateway_url()}/app/invoke/{app_id}", json={"request_data": payload}, stream=True, timeout=3600) as r:
        if r.status_code != 200:
            print(f"{r.status_code}: {r.text}", file=sys.stderr)
            return 1
        if r.headers.get("content-type", "").startswith("application/json"):
            data = r.json()
            if a.png_key:
                print(f"image written to {save_png(extract_nested(data, a.png_key), a.save_png_path)}")
                data = {k: v for k, v in data.items() if k != a.png_key.split('.')[0]} if isinstance(data, dict) else data
            print(json.dumps(data, indent=1))
            return 0
        aggregated: dict[str, list[str]] = {k: [] for k in a.aggregate_keys}
        for line in r.iter_lines():
            if not line:
                continue
            chunk = json.loads(line)
            if isinstance(chunk, dict) and "error" in chunk and len(chunk) == 1:
                print(f"error: {chunk['error']}", file=sys.stderr)
                return 1
            if player is not None:
                val = extract_nested(chunk, a.audio_key)
                if val:
                    player.feed(base64.b64decode(val))
            if a.aggregate_keys:
                for k in a.aggregate_keys:
                    val = extract_nested(chunk, k)
                    if isinstance(val, str):
                        aggregated[k].append(val)
                        sys.stdout.write(val)
                        sys.stdout.flush()
            elif player is None:
                print(json.dumps(chunk))
        if a.aggregate_keys:
            print()
        if player is not None:
            player.close()
            if a.save_audio_path:
                player.save_wav(a.save_audio_path)
                print(f"audio written to {a.save_audio_path} ({len(player.collected)} bytes of PCM)")
    return 0


def cmd_tasklib(a: argparse.Namespace) -> int:
    if a.action == "purge":
        r = requests.post(f"{gateway_url()}/purge-tasklib", timeout=120)
        print("task library purged" if r.status_code == 200 else f"{r.status_code}: {r.text}")
        return 0 if r.status_code == 200 else 1
    from .tasklib_explorer import discover_tasklib

    req = discover_tasklib(a.target)
    print(f"uploading {len(req.task_definitions)} task classes and {len(req.descriptor_definitions)} descriptors")
    r = requests.post(f"{gateway_url()}/deploy-tasks", json=req.model_dump(), timeout=300)
    print(r.json() if r.status_code == 200 else f"{r.status_code}: {r.text}")
    return 0 if r.status_code == 200 else 1


def cmd_deploy_profiles(a: argparse.Namespace) -> int:
    profiles = []
    for f in sorted(Path(a.dir).glob("*.json")):
        d = json.loads(f.read_text())
        if "task" not in d or "num_gpus_to_profile" not in d:
            print(f"skipping {f.name}: not a unit-task profile", file=sys.stderr)
            continue
        profiles.append(d)
        print(f"{f.name}: GPUs per executor {sorted(int(k) for k in d['num_gpus_to_profile'])}")
    if a.dry_run:
        print(f"{len(profiles)} profiles valid (dry run, nothing sent)")
        return 0
    r = requests.post(f"{gateway_url()}/deploy-profiles", json={"profiles": profiles}, timeout=120)
    print(r.json() if r.status_code == 200 else f"{r.status_code}: {r.text}")
    return 0 if r.status_code == 200 else 1


def cmd_scale(a: argparse.Namespace) -> int:
    r = requests.post(f"{gateway_url()}/task/scale", json={"task_id": a.task_id, "num_gpus": a.num_gpus}, timeout=1800)
    print("ok" if r.status_code == 200 else f"{r.status_code}: {r.text}")
    return 0 if r.status_code == 200 else 1


def cmd_up(a: argparse.Namespace) -> int:
    from ..services.local_cluster import run_forever

    run_forever(num_gpus=a.num_gpus, cpu=a.cpu, gateway_port=a.port)
    return 0


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="cornserve", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("up"); s.add_argument("--num-gpus", type=int, default=None); s.add_argument("--cpu", action="store_true")
    s.add_argument("--port", type=int, default=None); s.set_defaults(fn=cmd_up)
    s = sub.add_parser("register"); s.add_argument("path"); s.add_argument("--alias"); s.add_argument("--no-logs", action="store_true")
    s.set_defaults(fn=cmd_register)
    s = sub.add_parser("unregister"); s.add_argument("app"); s.set_defaults(fn=cmd_unregister)
    s = sub.add_parser("list"); s.set_defaults(fn=cmd_list)
    s = sub.add_parser("invoke"); s.add_argument("app"); s.add_argument("data")
    s.add_argument("--aggregate-keys", nargs="*", default=[]); s.add_argument("--png-key"); s.add_argument("--save-png-path")
    s.add_argument("--audio-key"); s.add_argument("--save-audio-path"); s.add_argument("--sample-rate", type=int, default=24000)
    s.add_argument("--no-play", action="store_true"); s.set_defaults(fn=cmd_invoke)
    s = sub.add_parser("tasklib"); s.add_argument("action", choices=["deploy", "purge"]); s.add_argument("target", nargs="?", default="")
    s.set_defaults(fn=cmd_tasklib)
    s = sub.add_parser("deploy_profiles"); s.add_argument("dir"); s.add_argument("--dry-run", action="store_true")
    s.set_defaults(fn=cmd_deploy_profiles)
    s = sub.add_parser("scale"); s.add_argument("task_id"); s.add_argument("num_gpus", type=int); s.set_defaults(fn=cmd_scale)
    return p


def main(argv: list[str] | None = None) -> None:
    args = build_parser().parse_args(argv)
    sys.exit(args.fn(args))


if __name__ == "__main__":
    main()
