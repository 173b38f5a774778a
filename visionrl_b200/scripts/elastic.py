"""Restart a multi-rank training run in place after a rank failed.

    torchrun --nproc-per-node 8 -m vrl.scripts.elastic --max-restarts 2 \
        --config experiment/<name> [key=value ...]

Failure handling in this package ends a job cleanly instead of hanging it: a rank whose step
raises announces it through the rendezvous store, its peers learn of it before their next launch
(``visionrl_b200.parallel.liveness``) or their next collective fails, and every device-side wait
is bounded.  What follows a failure is the reference's recovery too — start again from the last
``checkpoint.pt`` (``vrl/trainers/checkpointing.py``) — and there are two ways to get it:

* the processes died: let the launcher start new ones (``torchrun --max-restarts N``) with
  ``trainer.resume_from=auto``, which picks the latest complete checkpoint below
  ``trainer.output_dir`` and starts fresh when there is none;
* the processes are alive (a software error on one rank, a peer that fell silent, a collective
  that timed out): this module.  Every rank catches the failure, leaves the old process group
  without a barrier, moves to the next rendezvous port, forms a new group and runs the recipe
  again with ``trainer.resume_from=auto``.  All ranks count attempts the same way, so they meet
  at the same port without talking to each other.

Rendezvous of a restart.  Under ``torchrun`` the launcher's agent keeps one key-value store
alive for the whole job and every rank is a client of it; the new group uses that store under a
per-attempt key prefix, so nothing written by the group that was left (addresses, heartbeats,
failure notices) is read again.  Without an agent store rank 0 hosts the store, and attempt ``k``
moves to ``ports[k]`` when a list is given (``--ports a,b,c`` or ``VRL_ELASTIC_PORTS``), else to
``MASTER_PORT + k``.  A rank may arrive at the rendezvous long before the others (the rank that
failed leaves at once, a survivor may first sit out its collective's time-out), so the rendezvous
waits ``rendezvous_timeout_s`` (default ten minutes), independently of the collectives' time-out.

Nothing here runs on a GPU by itself; the restart decision, the teardown and the rendezvous are
host code, exercised by the tests on CPU ranks.
"""

from __future__ import annotations

import argparse
import asyncio
import inspect
import logging
import os
import sys
from typing import Any, Callable, Sequence

from visionrl_b200.parallel.mesh import agent_store_in_use

logger = logging.getLogger(__name__)

# errors that the same command line would hit again: restarting cannot help
_FATAL = (KeyboardInterrupt, SystemExit, GeneratorExit, FileNotFoundError, ImportError, SyntaxError,
          TimeoutError)


def _world_size() -> int:
    try:
        return int(os.environ.get("WORLD_SIZE", "1"))
    except ValueError:
        return 1


def _leave_group() -> None:
    """Drop this rank's side of the process group; no barrier, the peers may be gone."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - a half-open group must not stop the restart
        logger.debug("process group teardown failed", exc_info=True)
    try:
        from visionrl_b200.parallel import mesh as mesh_module

        mesh_module._CURRENT[0] = None
    except Exception:  # noqa: BLE001
        pass


def restart_store_factory(attempt: int, rendezvous_timeout_s: float) -> Callable[[int, int], Any]:
    """The store of restart ``attempt``, under a key prefix of its own."""

    def factory(rank: int, world: int) -> Any:
        from visionrl_b200.parallel.mesh import fresh_prefix_store

        relaunches = int(os.environ.get("TORCHELASTIC_RESTART_COUNT") or 0)
        return fresh_prefix_store(rank, world, f"vrl/restart/{relaunches}.{attempt}", rendezvous_timeout_s)

    return factory


def _clear_store_factory() -> None:
    from visionrl_b200.parallel.mesh import set_rendezvous_store_factory

    set_rendezvous_store_factory(None)


def rendezvous_port(attempt: int, ports: Sequence[int] | None, base_port: int) -> int:
    if ports:
        if attempt >= len(ports):
            raise ValueError(f"attempt {attempt} needs a rendezvous port but only {len(ports)} were given")
        return int(ports[attempt])
    return int(base_port) + int(attempt)


def restartable(exc: BaseException, *, group_was_formed: bool) -> bool:
    """A failure is worth a restart when the job had got as far as forming its process group
    (what fails before that — a config that does not validate, a missing manifest — fails the
    same way again) and it is not one of the errors no restart can cure."""
    if isinstance(exc, _FATAL):
        return False
    return group_was_formed and isinstance(exc, Exception)


def run_with_restarts(config: str, overrides: Sequence[str] = (), *, max_restarts: int = 2,
                      ports: Sequence[int] | None = None, rendezvous_timeout_s: float = 600.0,
                      before_attempt: Callable[[int], Any] | None = None) -> tuple[Any, int]:
    """Run the recipe ``config`` names; after a restartable failure of a multi-rank job leave the
    process group, move to the next rendezvous port and run it again from the latest checkpoint.
    Returns ``(recipe result, restarts used)``.  ``before_attempt(k)`` is called at the start of
    attempt ``k`` (tests inject their failure there)."""
    from visionrl_b200.config.loader import load_config
    from visionrl_b200.scripts.train import run_config

    if max_restarts < 0:
        raise ValueError("max_restarts must be >= 0")
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    attempt = 0
    while True:
        if _world_size() > 1 and attempt > 0:
            from visionrl_b200.parallel.mesh import set_rendezvous_store_factory

            if not agent_store_in_use():
                os.environ["MASTER_PORT"] = str(rendezvous_port(attempt, ports, base_port))
            set_rendezvous_store_factory(restart_store_factory(attempt, rendezvous_timeout_s))
        os.environ["VRL_RESTART_ATTEMPT"] = str(attempt)
        extra = ["trainer.resume_from=auto"] if attempt > 0 else []
        if before_attempt is not None:
            before_attempt(attempt)
        formed = False
        try:
            cfg = load_config(config, overrides=[*overrides, *extra])
            outcome = run_config(cfg)
            if inspect.isawaitable(outcome):
                loop = asyncio.new_event_loop()
                try:
                    outcome = loop.run_until_complete(outcome)
                finally:
                    loop.close()
            _clear_store_factory()
            return outcome, attempt
        except BaseException as exc:
            _clear_store_factory()
            try:
                import torch.distributed as dist

                formed = dist.is_available() and dist.is_initialized()
            except Exception:  # noqa: BLE001
                formed = False
            _leave_group()
            if attempt >= max_restarts or not restartable(exc, group_was_formed=formed):
                raise
            attempt += 1
            logger.warning("attempt %d failed (%s: %s); restarting from the latest checkpoint, "
                           "restart %d of %d", attempt - 1, type(exc).__name__, exc, attempt, max_restarts)


def _parse_ports(text: str | None) -> list[int] | None:
    if not text:
        return None
    return [int(p) for p in text.replace(" ", "").split(",") if p]


def main(argv: list[str] | None = None) -> int:
    from visionrl_b200.scripts.train import _configure_logging, _launcher_rank

    rank, world = _launcher_rank()
    _configure_logging(rank, world)
    parser = argparse.ArgumentParser(
        prog="vrl-elastic", description="Run a training recipe and restart it in place, from the "
                                        "latest checkpoint, when a rank fails.")
    parser.add_argument("--config", required=True)
    parser.add_argument("--max-restarts", type=int, default=2)
    parser.add_argument("--ports", default=os.environ.get("VRL_ELASTIC_PORTS"),
                        help="comma-separated rendezvous ports, one per attempt "
                             "(default: MASTER_PORT, MASTER_PORT+1, ...)")
    parser.add_argument("--rendezvous-timeout", type=float, default=600.0,
                        help="seconds a restarted rank waits for the others to arrive")
    parser.add_argument("overrides", nargs="*", metavar="key=value")
    args = parser.parse_args(argv)
    try:
        _, restarts = run_with_restarts(args.config, args.overrides, max_restarts=args.max_restarts,
                                        ports=_parse_ports(args.ports),
                                        rendezvous_timeout_s=args.rendezvous_timeout)
        if restarts:
            logger.info("finished after %d restart(s)", restarts)
    finally:
        _leave_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
