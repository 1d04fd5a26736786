"""Input-pipeline throughput: JPEG records -> normalised fp16 NHWC training batches on the GPU.

Two arms over the same RecordIO file of synthetic 500 x 375 JPEG images (the typical ImageNet size):
``host``: `ImageRecordIter` decoding and augmenting on `--threads` host threads, float batch copied to the device;
``gpu``:  `ImageRecordIter(device=gpu)`: nvJPEG decode and the one-kernel augmentation on the device.
Prints one JSON line per arm with images/s (wall clock over whole epochs after a warm-up epoch; the device is synchronised
before the clock is read).

    python benchmark/image_pipeline.py --images 512 --batch 128 --epochs 3
"""
import argparse
import io
import json
import os
import sys
import tempfile
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--images', type=int, default=512)
    ap.add_argument('--batch', type=int, default=128)
    ap.add_argument('--epochs', type=int, default=3)
    ap.add_argument('--threads', type=int, default=8)
    args = ap.parse_args()
    import torch
    from PIL import Image
    import mxnet_b200 as mx
    from mxnet_b200 import recordio
    rng = np.random.RandomState(0)
    path = os.path.join(tempfile.mkdtemp(), 'bench.rec')
    w = recordio.MXRecordIO(path, 'w')
    yy, xx = np.mgrid[0:375, 0:500].astype('float32')
    nbytes = 0
    for i in range(args.images):
        img = np.stack([127 + 90 * np.sin(yy / rng.uniform(5, 40)) * np.cos(xx / rng.uniform(5, 40)) + rng.randn(375, 500) * 12
                        for _ in range(3)], -1)
        b = io.BytesIO()
        Image.fromarray(np.clip(img, 0, 255).astype('uint8')).save(b, format='JPEG', quality=90)
        nbytes += len(b.getvalue())
        w.write(recordio.pack(recordio.IRHeader(0, float(i % 1000), i, 0), b.getvalue()))
    w.close()
    kw = dict(path_imgrec=path, data_shape=(3, 224, 224), batch_size=args.batch, resize=256, rand_crop=True, rand_mirror=True,
              mean_r=123.68, mean_g=116.28, mean_b=103.53, std_r=58.4, std_g=57.1, std_b=57.4, layout='NHWC',
              preprocess_threads=args.threads)
    ctx = mx.gpu(0)
    for arm in ('host', 'gpu'):
        it = mx.io.ImageRecordIter(device=ctx, dtype='float16', **kw) if arm == 'gpu' else mx.io.ImageRecordIter(**kw)
        n = 0
        for epoch in range(args.epochs + 1):
            if epoch == 1:
                torch.cuda.synchronize()
                t0, n = time.time(), 0
            it.reset()
            for batch in it:
                x = batch.data[0]
                if arm == 'host':
                    x = x.as_in_context(ctx).astype('float16')
                n += x.shape[0] - batch.pad
        torch.cuda.synchronize()
        dt = time.time() - t0
        print(json.dumps({'arm': arm, 'images_per_s': round(n / dt, 1), 'images': n, 'seconds': round(dt, 3),
                          'mean_jpeg_bytes': nbytes // args.images, 'batch': args.batch,
                          'host_threads': args.threads if arm == 'host' else 0}), flush=True)


if __name__ == '__main__':
    main()
