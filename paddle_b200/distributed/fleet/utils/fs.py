"""File-system clients (python/paddle/distributed/fleet/utils/fs.py: ``FS`` :60, ``LocalFS`` :119, ``HDFSClient``
:462, ``AFSClient`` :1239).  Only the local client is functional; the HDFS / AFS clients shell out to cluster tools
that do not exist here and raise at construction."""
from __future__ import annotations

import os
import shutil


class ExecuteError(Exception):
    pass


class FSFileExistsError(Exception):
    pass


class FSFileNotExistsError(Exception):
    pass


class FSTimeOut(Exception):
    pass


class FSShellCmdAborted(ExecuteError):
    pass


class FS:
    pass


class LocalFS(FS):
    def ls_dir(self, fs_path):
        if not self.is_exist(fs_path):
            return [], []
        dirs, files = [], []
        for f in os.listdir(fs_path):
            (dirs if os.path.isdir(os.path.join(fs_path, f)) else files).append(f)
        return dirs, files

    def list_dirs(self, fs_path):
        return self.ls_dir(fs_path)[0]

    def list_files_info(self, fs_path):
        return [(f, os.path.getsize(os.path.join(fs_path, f))) for f in self.ls_dir(fs_path)[1]]

    def mkdirs(self, fs_path):
        assert not os.path.isfile(fs_path), f"{fs_path} is already a file"
        os.makedirs(fs_path, exist_ok=True)

    def rename(self, fs_src_path, fs_dst_path):
        os.rename(fs_src_path, fs_dst_path)

    def delete(self, fs_path):
        if not self.is_exist(fs_path):
            return
        if os.path.isfile(fs_path):
            os.remove(fs_path)
        else:
            shutil.rmtree(fs_path)

    def need_upload_download(self):
        return False

    def is_file(self, fs_path):
        return os.path.isfile(fs_path)

    def is_dir(self, fs_path):
        return os.path.isdir(fs_path)

    def is_exist(self, fs_path):
        return os.path.exists(fs_path)

    def touch(self, fs_path, exist_ok=True):
        if self.is_exist(fs_path):
            if exist_ok:
                return
            raise FSFileExistsError(fs_path)
        open(fs_path, "a").close()

    def mv(self, src_path, dst_path, overwrite=False, test_exists=False):
        if not self.is_exist(src_path):
            raise FSFileNotExistsError(src_path)
        if overwrite and self.is_exist(dst_path):
            self.delete(dst_path)
        if self.is_exist(dst_path):
            raise FSFileExistsError(dst_path)
        return self.rename(src_path, dst_path)

    def upload(self, local_path, fs_path, *a, **k):
        shutil.copy(local_path, fs_path)

    def download(self, fs_path, local_path, *a, **k):
        shutil.copy(fs_path, local_path)

    def cat(self, fs_path=None):
        with open(fs_path) as f:
            return f.read()


class HDFSClient(FS):
    def __init__(self, hadoop_home, configs, time_out=5 * 60 * 1000, sleep_inter=1000):
        raise NotImplementedError("HDFSClient drives the `hadoop fs` command line, which is not available; use LocalFS")


class AFSClient(FS):
    def __init__(self, time_out=5 * 60 * 1000, sleep_inter=1000):
        raise NotImplementedError("AFSClient needs the AFS runtime, which is not available; use LocalFS")
