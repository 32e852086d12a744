"""Discovery, server side: waits until somebody knocks
(tunix/experimental/distributed/examples/basics/door.py).

Run together with `knocker` as two logical processes of one launcher:

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process --process_main=tunix_b200.experimental.distributed.examples.basics.door.main \\
                --discovery_id=door --discovery_port=12345 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.basics.knocker.main \\
                --discovery_id=knocker --discovery_addrs=door:12345 --say="open up"

Metadata is opaque bytes to the discovery service; these two agree on UTF-8 text (nothing is unpickled from a peer).
"""
import argparse
import logging
import threading


def main(ctx, argv) -> str:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="this is door!")
  parser.add_argument("--wait_s", type=float, default=60.0)
  args = parser.parse_args(argv)
  logging.info(args.message)
  knocked = threading.Event()
  heard = []

  def on_knock(hostname: str, port: int, metadata: bytes) -> None:
    heard.append(f"{hostname} knocked and said: {metadata.decode('utf-8')}")
    logging.info(heard[-1])
    knocked.set()
  ctx.ipc.discovery.on_register(on_knock)
  if not knocked.wait(args.wait_s):
    raise SystemExit(f"nobody knocked within {args.wait_s:.0f} s")
  return heard[0]
