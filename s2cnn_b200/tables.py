"""Control of the library's constant tables (Wigner-d panels, FFT twiddles, quadrature weights).

Tables are built in float64 on the host the first time a bandwidth is used on a device and kept
for the life of the process (the reference: ``lru_cache`` on ``_setup_wigner``,
s2cnn/soft/so3_fft.py:205-209).  ``set_table_cache_dir`` additionally keeps the large Wigner tables
on disk between processes - the counterpart of the reference's ``cached_dirpklgz`` decorator
(s2cnn/utils/decorator.py:54-104), but with one checksummed file per table written atomically, so
that several processes (one per GPU) can share a directory.  A message is logged on the
``"trainer"`` logger whenever a table had to be computed rather than read, as the reference does
(s2cnn/soft/so3_fft.py:223)."""
import logging
import os

from . import _lib


def set_table_cache_dir(path):
    """Directory for the on-disk table cache (created if missing); ``None`` turns the cache off."""
    lib = _lib.cuda_lib()
    if path is None:
        lib.s2c_set_table_cache_dir(None)
        return
    os.makedirs(path, exist_ok=True)
    lib.s2c_set_table_cache_dir(os.fsencode(path))
    logging.getLogger("trainer").info("s2cnn_b200: Wigner tables are cached under %s", path)


def table_cache_counters():
    """(tables read from disk, tables written to disk) by this process."""
    lib = _lib.cuda_lib()
    return int(lib.s2c_table_cache_hits()), int(lib.s2c_table_cache_stores())


def clear_tables():
    """Frees the in-memory (device) tables of every GPU; they are rebuilt, or re-read from the disk
    cache, on next use."""
    _lib.cuda_lib().s2c_clear_tables()
