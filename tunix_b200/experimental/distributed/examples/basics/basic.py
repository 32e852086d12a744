"""The smallest process body for the runtime launcher
(tunix/experimental/distributed/examples/basics/basic.py).

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process_main=tunix_b200.experimental.distributed.examples.basics.basic.main

A body is `main(ctx, argv)`: `argv` holds the flags the launcher did not consume, `ctx` the platform-dependent
services (`ctx.dist` for the process group, `ctx.ipc.discovery` for finding peers).
"""
GREETING = "hello world"

main = lambda ctx, argv: print(GREETING)  # noqa: E731 - a body is any callable of (ctx, argv)
