__version__ = '0.1.0'
__release_datetime__ = '2026-11-25 00:00:00'
