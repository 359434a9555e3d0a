"""Worker for the 2-rank test of the drop-in surface (launched with torch.distributed.run): each
rank runs the same SONATA project through Config / PointNetwork / PointSimulator; rank 0 writes the
merged spikes and report files."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from bmtk_b200 import pointnet
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', '0')))
    dist.init_process_group('gloo')
    pointnet.io_tools.io.set_barrier(dist.barrier)
    conf = pointnet.Config.from_json(sys.argv[1])
    conf.build_env()
    net = pointnet.PointNetwork.from_config(conf)
    sim = pointnet.PointSimulator.from_config(conf, net)
    sim.run()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
