#!/usr/bin/env python
"""Write docker-compose.yml for N node containers and bring the cluster up (or down).

    python docker/compose_up.py --nodes 8            # generate + `docker compose up --build -d`
    python docker/compose_up.py --down               # `docker compose down`
    python docker/compose_up.py --nodes 4 --dry-run  # only write the file

The reference drives its benchmark clusters the same way (docker/compose_up.py:43-58)."""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=8)
    ap.add_argument("--base-port", type=int, default=40000)
    ap.add_argument("--rate", default=None, help="rate-limit the nodes' network (Pumba), e.g. 10mbit")
    ap.add_argument("--file", default=os.path.join(ROOT, "docker-compose.yml"))
    ap.add_argument("--down", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args()
    docker = shutil.which("docker")
    if a.down:
        if docker is None:
            print("docker is not installed on this machine", file=sys.stderr)
            return 1
        return subprocess.call([docker, "compose", "-f", a.file, "down"])
    cmd = [sys.executable, os.path.join(HERE, "gen_compose.py"), "--nodes", str(a.nodes), "--base-port", str(a.base_port)]
    if a.rate:
        cmd += ["--rate", a.rate]
    text = subprocess.run(cmd, check=True, capture_output=True, text=True)
    with open(a.file, "w") as f:
        f.write(text.stdout)
    sys.stderr.write(text.stderr)
    print(f"wrote {a.file}")
    if a.dry_run:
        return 0
    if docker is None:
        print("docker is not installed on this machine: the compose file is written, nothing was started", file=sys.stderr)
        return 1
    return subprocess.call([docker, "compose", "-f", a.file, "up", "--build", "-d"])


if __name__ == "__main__":
    sys.exit(main())
