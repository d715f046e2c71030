"""``python -m nangila.cli.dump ...``: runs the ``nangila-dump`` tool (built on first use).
Sub-commands: verify -c FILE | diff -a FILE -b FILE | inspect -c FILE [-o OUT] | info -c FILE
(reference tool: nangila-dump/src/main.rs)."""
import subprocess
import sys

from .. import _build


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    tools = {p.name: p for p in _build.build_cli()}
    return subprocess.call([str(tools["nangila-dump"]), *argv])


if __name__ == "__main__":
    sys.exit(main())
