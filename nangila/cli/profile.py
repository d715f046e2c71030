"""``python -m nangila.cli.profile ...``: runs the ``nangila-profile`` tool (built on first use).
Sub-commands: calibrate -g grads.jsonl [-s N] [-t T] -o MASK [--report JSON] | report -m MASK -o JSON |
info -m MASK (reference tool: nangila-profile/src/main.rs)."""
import subprocess
import sys

from .. import _build


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    tools = {p.name: p for p in _build.build_cli()}
    return subprocess.call([str(tools["nangila-profile"]), *argv])


if __name__ == "__main__":
    sys.exit(main())
