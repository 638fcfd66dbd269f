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
