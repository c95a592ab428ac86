"""``python -m kraken_b200.launch.ps_server --port 50001 --addr 127.0.0.1:50001 --s_addr 127.0.0.1:50000``

One parameter-server shard of the multi-process CPU deployment.  Flags as in
the reference's ps_server binary (kraken/executable/ps_server_main.cc:5-10);
``--thread_nums`` is accepted for compatibility (the server runs a thread per connection).
"""
import argparse
import logging
import os
import threading

from ..runtime.remote import PsServer


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--port", type=int, default=50001)
    p.add_argument("--thread_nums", type=int, default=2)
    p.add_argument("--addr", default="")
    p.add_argument("--s_addr", required=True)
    p.add_argument("--saved_dir", default="")
    p.add_argument("--max_save_count", type=int, default=3)
    a = p.parse_args(argv)
    from kraken_b200.utils.log import configure
    configure(os.environ.get("KRAKEN_LOG_LEVEL", "info"))
    s = PsServer(a.port, a.addr or f"127.0.0.1:{a.port}", a.s_addr, a.saved_dir, a.max_save_count)
    s.start()
    threading.Event().wait()


if __name__ == "__main__":
    main()
