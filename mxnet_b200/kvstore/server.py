"""Parameter server with the update semantics of the reference's distributed KVStore.

Reference: ``src/kvstore/kvstore_dist_server.h`` (``KVStoreDistServer::ApplyUpdates``, lines 349-404) over ps-lite.  A
server holds the stored value of every key and (optionally) an updater:

* **sync mode** (``dist_sync``): the pushes of one round are merged (summed) until every worker has pushed the key; then the
  updater runs once on the merged value (or, without an updater, the merged value replaces the stored one), and only then
  are that round's pushes acknowledged and its pulls answered;
* **async mode** (``dist_async``): every push is applied to the stored value immediately through the updater, with no
  waiting for other workers; a pull returns whatever the store holds at that moment.  An updater is required.

Here the server is a thread inside the process of rank 0 (there is no separate scheduler / server role to launch); workers
talk to it over one TCP connection each, with length-prefixed messages carrying the raw bytes of the arrays.  The address is
published through the job's rendezvous store.  Values live on the host in the server; the workers move them to and from
their devices.
"""
import pickle
import socket
import struct
import threading

import numpy as np
import torch

from ..base import MXNetError

__all__ = ['ParameterServer', 'ServerClient']


def _send(sock, obj):
    payload = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    sock.sendall(struct.pack('<Q', len(payload)) + payload)


def _recv_exact(sock, n):
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(n - len(buf), 1 << 20))
        if not chunk:
            raise ConnectionError('peer closed the connection')
        buf.extend(chunk)
    return bytes(buf)


def _recv(sock):
    (n,) = struct.unpack('<Q', _recv_exact(sock, 8))
    return pickle.loads(_recv_exact(sock, n))


def _to_wire(t):
    """(numpy array, torch dtype name): bfloat16 has no NumPy type and travels as float32."""
    t = t.detach().cpu()
    name = str(t.dtype).replace('torch.', '')
    return (t.float().numpy() if t.dtype == torch.bfloat16 else t.numpy()), name


def _from_wire(arr, name):
    t = torch.from_numpy(np.array(arr, copy=True))
    return t.to(getattr(torch, name)) if str(t.dtype) != 'torch.' + name else t


class ParameterServer(object):
    """The server side.  ``sync_mode`` selects merge-then-apply; otherwise every push is applied on arrival."""

    def __init__(self, num_workers, sync_mode, host='127.0.0.1', port=0):
        self.num_workers = int(num_workers)
        self.sync_mode = bool(sync_mode)
        self.store = {}                 # key -> torch tensor on the host
        self.updater = None
        self._merge = {}                # key -> [merged tensor, [connections waiting for the round]]
        self._lock = threading.Lock()
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((host, port))
        self._sock.listen(self.num_workers + 2)
        self.address = self._sock.getsockname()
        self._threads = []
        self._stopped = threading.Event()
        self._barrier_waiting = []
        self.pushes_applied = 0         # number of updater calls (observable by tests: async = one per push)
        self._accept_thread = threading.Thread(target=self._accept_loop, name='kvstore-server', daemon=True)
        self._accept_thread.start()

    # ---- connection handling -----------------------------------------------------------------------------------------------
    def _accept_loop(self):
        while not self._stopped.is_set():
            try:
                conn, _ = self._sock.accept()
            except OSError:
                return
            conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            t = threading.Thread(target=self._serve, args=(conn,), daemon=True)
            t.start()
            self._threads.append(t)

    def _serve(self, conn):
        try:
            while True:
                msg = _recv(conn)
                if not self._handle(conn, msg):
                    return
        except (ConnectionError, OSError):
            return
        finally:
            conn.close()

    # ---- requests ------------------------------------------------------------------------------------------------------------
    def _handle(self, conn, msg):
        op = msg[0]
        if op == 'init':
            _, key, arr, dtype = msg
            with self._lock:
                if key not in self.store:            # the first worker's value wins, as with rank 0 in the reference
                    self.store[key] = _from_wire(arr, dtype)
            _send(conn, ('ok',))
        elif op == 'set_optimizer':
            from ..optimizer.updater import get_updater
            with self._lock:
                if self.updater is None:
                    self.updater = get_updater(pickle.loads(msg[1]))
            _send(conn, ('ok',))
        elif op == 'push':
            _, key, arr, dtype, wants_pull = msg
            self._push(conn, key, _from_wire(arr, dtype), wants_pull)
        elif op == 'pull':
            _, key = msg
            with self._lock:
                if key not in self.store:
                    _send(conn, ('error', 'key %s has not been initialized' % str(key)))
                    return True
                value = _to_wire(self.store[key].clone())
            _send(conn, ('value',) + value)
        elif op == 'barrier':
            with self._lock:
                self._barrier_waiting.append(conn)
                release = self._barrier_waiting if len(self._barrier_waiting) == self.num_workers else None
                if release is not None:
                    self._barrier_waiting = []
            for c in release or ():
                _send(c, ('ok',))
        elif op == 'stats':
            with self._lock:
                _send(conn, ('stats', {'pushes_applied': self.pushes_applied, 'keys': len(self.store)}))
        elif op == 'stop':
            _send(conn, ('ok',))
            return False
        else:
            _send(conn, ('error', 'unknown request %r' % (op,)))
        return True

    def _apply(self, key, update):
        """One ``updater(key, update, stored)`` call, or a plain copy when no updater is installed (sync mode only)."""
        from ..ndarray.ndarray import NDArray
        stored = self.store[key]
        if self.updater is not None:
            self.updater(key, NDArray._from_tensor(update), NDArray._from_tensor(stored))
        else:
            stored.copy_(update)
        self.pushes_applied += 1

    def _push(self, conn, key, grad, wants_pull):
        with self._lock:
            if key not in self.store:
                _send(conn, ('error', 'key %s has not been initialized' % str(key)))
                return
            if not self.sync_mode:
                if self.updater is None:
                    _send(conn, ('error', 'Updater needs to be set for async mode'))
                    return
                self._apply(key, grad)
                reply = ('value',) + _to_wire(self.store[key].clone()) if wants_pull else ('ok',)
                _send(conn, reply)
                return
            slot = self._merge.get(key)
            if slot is None:
                slot = self._merge[key] = [grad.clone(), []]
            else:
                slot[0].add_(grad)
            slot[1].append((conn, wants_pull))
            if len(slot[1]) < self.num_workers:
                return                               # acknowledged when the round completes
            del self._merge[key]
            self._apply(key, slot[0])
            value = _to_wire(self.store[key].clone())
            waiting = slot[1]
        for c, pull in waiting:
            _send(c, ('value',) + value if pull else ('ok',))

    def stop(self):
        self._stopped.set()
        try:
            self._sock.close()
        except OSError:
            pass


class ServerClient(object):
    """A worker's connection to the server."""

    def __init__(self, address):
        self._sock = socket.create_connection(tuple(address))
        self._sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._lock = threading.Lock()

    def _call(self, *msg):
        with self._lock:
            _send(self._sock, msg)
            reply = _recv(self._sock)
        if reply[0] == 'error':
            raise MXNetError(reply[1])
        return reply

    def init(self, key, tensor):
        self._call('init', key, *_to_wire(tensor))

    def set_optimizer(self, optimizer):
        self._call('set_optimizer', pickle.dumps(optimizer))

    def push(self, key, tensor, pull=False):
        reply = self._call('push', key, *_to_wire(tensor), bool(pull))
        return _from_wire(reply[1], reply[2]) if reply[0] == 'value' else None

    def pull(self, key):
        reply = self._call('pull', key)
        return _from_wire(reply[1], reply[2])

    def barrier(self):
        self._call('barrier')

    def stats(self):
        return self._call('stats')[1]

    def close(self):
        try:
            self._call('stop')
        except Exception:   # pylint: disable=broad-except
            pass
        self._sock.close()
