"""Logging and rank helpers of the façade.

Same surface as the reference's IOUtils (bmtk/simulator/core/io_tools.py:39-134 and
bmtk/simulator/pointnet/io_tools.py:33-64): console + file logging on rank 0, `barrier()`,
`log_exception` = log on rank 0, barrier, raise. Rank and size come from the torchrun
environment (RANK / WORLD_SIZE) instead of nest.Rank()/NumProcesses().
"""
import logging
import os
import shutil
import sys


class IOUtils(object):
    def __init__(self):
        self.mpi_rank = int(os.environ.get('RANK', '0'))
        self.mpi_size = int(os.environ.get('WORLD_SIZE', '1'))
        self._log_format = logging.Formatter('%(asctime)s [%(levelname)s] %(message)s')
        self._log_level = logging.INFO
        self.log_to_console = True
        self._logger = None
        self._warned = set()
        self._barrier_fn = None

    @property
    def logger(self):
        if self._logger is None:
            self._logger = logging.getLogger('bmtk_b200.pointnet')
            self._logger.setLevel(self._log_level)
            self._logger.propagate = False
            if self.log_to_console and not any(isinstance(h, logging.StreamHandler) and not isinstance(h, logging.FileHandler)
                                               for h in self._logger.handlers):
                h = logging.StreamHandler(sys.stdout)
                h.setFormatter(self._log_format)
                self._logger.addHandler(h)
        return self._logger

    def set_log_format(self, fmt):
        self._log_format = logging.Formatter(fmt)

    def set_log_level(self, level):
        self._log_level = level if isinstance(level, int) else logging.getLevelName(level)
        if self._logger is not None:
            self._logger.setLevel(self._log_level)

    def set_barrier(self, fn):
        """Installs the collective used by barrier() (e.g. torch.distributed.barrier)."""
        self._barrier_fn = fn

    def barrier(self):
        if self._barrier_fn is not None and self.mpi_size > 1:
            self._barrier_fn()

    def quiet_simulator(self):
        pass

    def setup_output_dir(self, output_dir, log_file, overwrite=True):
        if self.mpi_rank == 0:
            if os.path.exists(output_dir):
                if overwrite:
                    shutil.rmtree(output_dir)
                    os.makedirs(output_dir)
                else:
                    self.log_warning('Directory {} already exists.'.format(output_dir))
            else:
                os.makedirs(output_dir)
        self.barrier()
        if log_file is not None:
            for h in [h for h in self.logger.handlers if isinstance(h, logging.FileHandler)]:
                self.logger.removeHandler(h)
                h.close()
            fh = logging.FileHandler(log_file)
            fh.setFormatter(self._log_format)
            self.logger.addHandler(fh)
            self.log_info('Created log file')

    def log_info(self, message, all_ranks=False):
        if all_ranks or self.mpi_rank == 0:
            self.logger.info(message)

    def log_warning(self, message, all_ranks=False, display_once=False):
        if not all_ranks and self.mpi_rank != 0:
            return
        if display_once and message in self._warned:
            return
        self._warned.add(message)
        self.logger.warning(message)

    def log_error(self, message):
        self.logger.error(message)

    def log_debug(self, message, all_ranks=False):
        if all_ranks or self.mpi_rank == 0:
            self.logger.debug(message)

    def log_exception(self, message, raise_exception=True):
        if self.mpi_rank == 0:
            self.logger.error(message)
        self.barrier()
        if raise_exception:
            raise Exception(message)


io = IOUtils()
