"""Role makers (python/paddle/distributed/fleet/base/role_maker.py): who this process is in the job.
Collective jobs only have workers; the environment variables are the launcher's (``PADDLE_TRAINER_ID``,
``PADDLE_TRAINERS_NUM``, ``PADDLE_TRAINER_ENDPOINTS``) with the torchrun names as fall-back."""
from __future__ import annotations

import os


class Role:
    WORKER = 1
    SERVER = 2
    HETER_WORKER = 3
    ALL = 4
    COORDINATOR = 5


class RoleMakerBase:
    def __init__(self):
        self._worker_endpoints, self._server_endpoints = [], []
        self._role, self._current_id, self._is_collective = Role.WORKER, 0, True

    def _is_worker(self):
        return self._role == Role.WORKER

    def _is_server(self):
        return self._role == Role.SERVER

    def _is_first_worker(self):
        return self._is_worker() and self._current_id == 0

    def _worker_num(self):
        return max(len(self._worker_endpoints), self._trainers_num)

    def _server_num(self):
        return len(self._server_endpoints)

    def _worker_index(self):
        return self._current_id

    def _server_index(self):
        return self._current_id

    def _role_id(self):
        return self._current_id

    def _node_num(self):
        return max(len({e.split(":")[0] for e in self._worker_endpoints}), 1)

    def _get_trainer_endpoints(self):
        return self._worker_endpoints

    def _get_pserver_endpoints(self):
        return self._server_endpoints

    def to_string(self):
        return f"role: {self._role}, current_id: {self._current_id}, worker_endpoints: {self._worker_endpoints}"

    # public aliases used by older scripts
    is_worker, is_server, is_first_worker = _is_worker, _is_server, _is_first_worker
    worker_num, worker_index, server_num, server_index = _worker_num, _worker_index, _server_num, _server_index


class PaddleCloudRoleMaker(RoleMakerBase):
    def __init__(self, is_collective=False, **kwargs):
        super().__init__()
        self._is_collective = is_collective
        self._kwargs = kwargs
        env = os.environ
        self._current_id = int(env.get("PADDLE_TRAINER_ID", env.get("RANK", 0)))
        self._trainers_num = int(env.get("PADDLE_TRAINERS_NUM", env.get("WORLD_SIZE", 1)))
        eps = env.get("PADDLE_TRAINER_ENDPOINTS", "")
        self._worker_endpoints = [e for e in eps.split(",") if e]
        self._server_endpoints = [e for e in env.get("PADDLE_PSERVERS_IP_PORT_LIST", "").split(",") if e]
        role = env.get("TRAINING_ROLE", "TRAINER")
        self._role = Role.SERVER if role == "PSERVER" and not is_collective else Role.WORKER

    def _generate_role(self):
        return self


class UserDefinedRoleMaker(PaddleCloudRoleMaker):
    def __init__(self, is_collective=False, init_gloo=False, current_id=0, role=Role.WORKER, worker_num=1,
                 worker_endpoints=None, server_endpoints=None, **kwargs):
        RoleMakerBase.__init__(self)
        self._is_collective, self._kwargs = is_collective, kwargs
        self._current_id, self._role = current_id, role
        self._worker_endpoints = list(worker_endpoints or [])
        self._server_endpoints = list(server_endpoints or [])
        self._trainers_num = worker_num or len(self._worker_endpoints)
