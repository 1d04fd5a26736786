"""``mx.kv`` / ``mx.kvstore``."""
from .base import KVStoreBase, TestStore, create
from .kvstore import KVStore
from .horovod import Horovod
from .byteps import BytePS
from .kvstore_server import KVStoreServer
from .gradient_compression import GradientCompression
