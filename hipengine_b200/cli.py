"""``hipengine-b200`` command line: ``serve`` / ``router`` / ``chat`` / ``bench`` / ``version``
(the reference's ``hipengine serve / chat / bench / version``, ``hipengine/cli.py:21-104``)."""
from __future__ import annotations

import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: hipengine-b200 {serve,router,chat,bench [micro|serving|prefill-stages],build,version} [options]")
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "version":
        from . import __version__
        print(__version__)
        return 0
    if cmd == "serve":
        from .server.__main__ import main as serve_main
        return serve_main(rest)
    if cmd == "router":
        from .server.router import main as router_main
        return router_main(rest)
    if cmd == "chat":
        from .chat_cli import main as chat_main
        return chat_main(rest)
    if cmd == "build":
        from .core import build
        print(build.build(verbose="-v" in rest))
        return 0
    if cmd == "bench":
        # bench [micro] KERNEL ... | bench serving ... | bench prefill-stages ...
        kind = rest[0] if rest and rest[0] in ("micro", "serving", "prefill-stages") else "micro"
        args = rest[1:] if rest and rest[0] == kind else rest
        if kind == "serving":
            from .benchmark.serving_load import main as serving_main
            return serving_main(args)
        if kind == "prefill-stages":
            from .benchmark import prefill_stages
            sys.argv = ["prefill_stages"] + args
            prefill_stages.main()
            return 0
        from .benchmark import micro
        sys.argv = ["micro"] + args
        micro.main()
        return 0
    print(f"unknown command {cmd!r}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
