"""Environment handed to the ranks (role of bluefog/run/env_util.py:25-76)."""
import re

# Variables that must not leak from the launcher's shell into the ranks.
_IGNORE = re.compile(r"^(BASH_FUNC_.*|OLDPWD|_|RANK|LOCAL_RANK|WORLD_SIZE|LOCAL_WORLD_SIZE)$")


def is_exportable(name: str) -> bool:
    return _IGNORE.match(name) is None


def rank_environment(environ, timeline=None, verbose=False):
    env = {k: v for k, v in environ.items() if is_exportable(k)}
    if timeline:
        env["BLUEFOG_TIMELINE"] = str(timeline)
    if verbose:
        env["BLUEFOG_LOG_LEVEL"] = "debug"
    return env
