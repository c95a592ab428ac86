"""``python -m kraken_b200.launch.scheduler_server --port 50000``

The control-plane process of the multi-process CPU deployment: membership ring,
table registry, save / load orchestration.  Same flag as the reference's
scheduler_server binary (kraken/executable/scheduler_server_main.cc:5).
"""
import argparse
import logging
import os
import threading

from ..runtime.remote import SchedulerServer


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--port", type=int, default=50000)
    a = p.parse_args(argv)
    from kraken_b200.utils.log import configure
    configure(os.environ.get("KRAKEN_LOG_LEVEL", "info"))
    s = SchedulerServer(a.port)
    s.start()
    logging.getLogger("kraken_b200").info("scheduler listening on port %d", s.port)
    threading.Event().wait()


if __name__ == "__main__":
    main()
