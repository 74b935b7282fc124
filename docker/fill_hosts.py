#!/usr/bin/env python
"""Print (or write) the hosts block that maps `node-<i>` to an address, so that a training.json written for the
compose network (`"addrs": ["node-0:40000", ...]`) also resolves from the host
(the reference's docker/fill_hosts.py:10-65 edits /etc/hosts the same way).

    python docker/fill_hosts.py --nodes 8                      # print the block
    python docker/fill_hosts.py --nodes 8 --write /etc/hosts   # replace the marked block in that file (needs the rights)
"""
import argparse
import re
import sys

BEGIN, END = "# >>> ono nodes >>>", "# <<< ono nodes <<<"


def block(nodes: int, ip: str) -> str:
    lines = [BEGIN] + [f"{ip}\tnode-{i}" for i in range(nodes)] + [END]
    return "\n".join(lines) + "\n"


def replace_block(text: str, new: str) -> str:
    pat = re.compile(re.escape(BEGIN) + r".*?" + re.escape(END) + r"\n?", re.S)
    if pat.search(text):
        return pat.sub(new, text)
    return text + ("" if text.endswith("\n") or not text else "\n") + new


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=8)
    ap.add_argument("--ip", default="127.0.0.1", help="address the published ports listen on")
    ap.add_argument("--write", default=None, help="file to update in place (default: print only)")
    a = ap.parse_args()
    new = block(a.nodes, a.ip)
    if not a.write:
        sys.stdout.write(new)
        return 0
    with open(a.write) as f:
        text = f.read()
    with open(a.write, "w") as f:
        f.write(replace_block(text, new))
    print(f"updated {a.write}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
