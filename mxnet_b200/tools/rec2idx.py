"""Rebuild the index of a RecordIO file:  python -m mxnet_b200.tools.rec2idx data.rec data.idx

Walks the records sequentially and writes ``key<TAB>byte offset`` lines, the key being the record's position (the
reference's tools/rec2idx.py does the same through MXRecordIOReaderTell)."""
import sys


def build_index(rec_path, idx_path):
    from .. import recordio
    reader = recordio.MXRecordIO(rec_path, 'r')
    n = 0
    with open(idx_path, 'w') as out:
        while True:
            pos = reader.tell()
            if reader.read() is None:
                break
            out.write('%d\t%d\n' % (n, pos))
            n += 1
    reader.close()
    return n


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    print('%d records' % build_index(argv[0], argv[1]))
    return 0


if __name__ == '__main__':
    sys.exit(main())
