"""Small helpers around the native extension (role of bluefog/common/util.py:30-53 in the reference)."""
import glob
import os


def extension_path(pkg_dir: str, name: str = "_C"):
    """Path of the built extension module ``name`` inside ``pkg_dir``, or None when it has not been built."""
    hits = sorted(glob.glob(os.path.join(pkg_dir, name + ".*.so")) + glob.glob(os.path.join(pkg_dir, name + ".so")))
    return hits[0] if hits else None


def check_extension(ext_name: str = "bluefog_b200", pkg_dir: str = None, name: str = "_C") -> None:
    """Raises ImportError when the native extension has not been built (``python setup.py build_ext --inplace``)."""
    pkg_dir = pkg_dir or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if extension_path(pkg_dir, name) is None:
        raise ImportError("Extension {} has not been built: run `python setup.py build_ext --inplace`.".format(ext_name))


def get_ext_suffix() -> str:
    """File-name suffix of extension modules for the running interpreter (``.cpython-312-x86_64-linux-gnu.so``);
    same contract as the reference's ``get_ext_suffix`` (bluefog/common/util.py:28-39)."""
    import sysconfig
    return sysconfig.get_config_var("EXT_SUFFIX") or sysconfig.get_config_var("SO") or ".so"


def get_extension_full_path(pkg_path: str, *names: str) -> str:
    """``<directory of pkg_path>/<names...><extension suffix>`` (bluefog/common/util.py:42-46)."""
    if not names:
        raise ValueError("at least the module name is needed")
    return os.path.join(os.path.dirname(pkg_path), *names[:-1], names[-1] + get_ext_suffix())


def is_running_from_ipython() -> bool:
    """True inside an IPython/Jupyter kernel (the interactive launcher's notebooks)."""
    try:
        from IPython import get_ipython
    except ImportError:
        return False
    return get_ipython() is not None


class env:
    """``with env(BLUEFOG_TIMELINE="/tmp/t", OTHER=None):`` sets the given environment variables for the body and puts
    the previous values (or absence) back afterwards; arguments that are None are ignored.  Also usable as a
    decorator-free plain object: ``e = env(A="1"); e.__enter__(); ...; e.__exit__()``.  Contract of the reference's
    context manager (bluefog/common/util.py:112-136)."""

    def __init__(self, **kwargs):
        self._new = {k: str(v) for k, v in kwargs.items() if v is not None}
        self._old = {}

    def __enter__(self):
        for k, v in self._new.items():
            self._old[k] = os.environ.get(k)
            os.environ[k] = v
        return self

    def __exit__(self, *exc):
        for k, old in self._old.items():
            if old is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = old
        self._old = {}
        return False
