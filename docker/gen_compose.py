#!/usr/bin/env python
"""Generate a docker-compose file with N identical node services, one GPU each, ports 40000+i
(the reference's docker/gen_compose.py:44-151 generates N one-CPU containers the same way).

    python docker/gen_compose.py --nodes 8 > docker-compose.yml && docker compose up --build

The printed `addrs` line is what goes into training.json."""
import argparse
import sys

SERVICE = """  node-{i}:
    build:
      context: .
      dockerfile: docker/Dockerfile
    environment:
      - PORT={port}
      - HOST=0.0.0.0
      - ONO_LOG={log}
    ports:
      - "{port}:{port}"
    ipc: host
    ulimits:
      memlock: -1
    deploy:
      resources:
        reservations:
          devices:
            - driver: nvidia
              device_ids: ["{i}"]
              capabilities: [gpu]
"""


# Optional traffic shaping of the control plane, as the reference's benchmark clusters do with Pumba
# (docker/gen_compose.py:15-41: `netem --duration ... rate 10mbit` on every node container). It touches the
# containers' TCP interfaces only; gradients between GPUs travel over NVLink and are not shaped.
PUMBA = """  pumba:
    image: gaiaadm/pumba
    volumes:
      - /var/run/docker.sock:/var/run/docker.sock
    command: netem --duration {duration} --tc-image gaiadocker/iproute2 rate --rate {rate} {targets}
    depends_on: [{deps}]
"""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=8)
    ap.add_argument("--base-port", type=int, default=40000)
    ap.add_argument("--log", default="info")
    ap.add_argument("--rate", default=None, help="shape every node's network to this rate with a Pumba container, e.g. 10mbit")
    ap.add_argument("--rate-duration", default="24h")
    a = ap.parse_args()
    out = ["services:"]
    for i in range(a.nodes):
        out.append(SERVICE.format(i=i, port=a.base_port + i, log=a.log))
    if a.rate:
        names = [f"node-{i}" for i in range(a.nodes)]
        out.append(PUMBA.format(duration=a.rate_duration, rate=a.rate, targets=" ".join(names), deps=", ".join(names)))
    sys.stdout.write("\n".join(out))
    addrs = ", ".join(f'"node-{i}:{a.base_port + i}"' for i in range(a.nodes))
    print(f"# addrs for training.json (from a container on the same network): [{addrs}]", file=sys.stderr)
    print("# note: GPUs in separate containers exchange gradients over NVLink only when the containers share the host IPC "
          "namespace (ipc: host) and see each other's devices; one container with all GPUs and "
          "`python -m oxidized_neural_orchestra_b200.runtime.launch` is the simpler bring-up on one box.", file=sys.stderr)


if __name__ == "__main__":
    main()
