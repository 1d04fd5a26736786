"""Callbacks for interactive training (``python/mxnet/notebook/callback.py``).

``PandasLogger`` collects per-batch, per-evaluation and per-epoch metrics into ``pandas.DataFrame`` tables; the
``Live*`` charts draw them with bokeh when that package is importable and are silent collectors otherwise.  The
callbacks take the ``BatchEndParam``-style object used by ``mx.callback`` (fields ``epoch``, ``nbatch``,
``eval_metric``)."""
import datetime
import time

try:
    import pandas as pd
except ImportError:      # pragma: no cover
    pd = None

try:
    import bokeh.plotting as _bokeh_plotting
    import bokeh.io as _bokeh_io
except ImportError:
    _bokeh_plotting = _bokeh_io = None


def _metric_pairs(param):
    metric = getattr(param, 'eval_metric', None)
    if metric is None:
        return []
    if hasattr(metric, 'get_name_value'):
        return list(metric.get_name_value())
    name, value = metric.get()
    if isinstance(name, (list, tuple)):
        return list(zip(name, value))
    return [(name, value)]


class PandasLogger(object):
    """Logs statistics about the training run into three tables: ``train`` (every ``frequent`` batches), ``eval``
    (every evaluation) and ``epoch`` (duration of every epoch)."""

    def __init__(self, batch_size, frequent=50):
        if pd is None:
            raise ImportError('PandasLogger needs pandas')
        self.batch_size, self.frequent = batch_size, frequent
        self._dataframes = {'train': pd.DataFrame(), 'eval': pd.DataFrame(), 'epoch': pd.DataFrame()}
        self.last_time = time.time()
        self.start_time = datetime.datetime.now()
        self.last_epoch_time = datetime.datetime.now()

    @property
    def train_df(self):
        return self._dataframes['train']

    @property
    def eval_df(self):
        return self._dataframes['eval']

    @property
    def epoch_df(self):
        return self._dataframes['epoch']

    @property
    def all_dataframes(self):
        return self._dataframes

    def elapsed(self):
        return datetime.datetime.now() - self.start_time

    def append_metrics(self, metrics, df_name):
        """Append one row (a dict of column -> value) to the table ``df_name``."""
        df = self._dataframes[df_name]
        row = pd.DataFrame([metrics], index=[len(df)])
        self._dataframes[df_name] = pd.concat([df, row], sort=False) if len(df) else row

    def train_cb(self, param):
        if param.nbatch % self.frequent == 0:
            self._process_batch(param, 'train')

    def eval_cb(self, param):
        self._process_batch(param, 'eval')

    def _process_batch(self, param, df_name):
        now = time.time()
        row = dict(_metric_pairs(param))
        if df_name == 'train':
            dt = max(now - self.last_time, 1e-9)
            row['batches_per_sec'] = self.frequent / dt
            row['records_per_sec'] = self.frequent * self.batch_size / dt
        row.update(elapsed=self.elapsed(), minibatch_count=param.nbatch, epoch=param.epoch)
        self.append_metrics(row, df_name)
        self.last_time = now

    def epoch_cb(self, *_args):
        now = datetime.datetime.now()
        self.append_metrics({'elapsed': self.elapsed(), 'epoch_time': now - self.last_epoch_time}, 'epoch')
        self.last_epoch_time = now

    def callback_args(self):
        """Keyword arguments for a ``fit``-style loop."""
        return {'batch_end_callback': self.train_cb, 'eval_end_callback': self.eval_cb, 'epoch_end_callback': self.epoch_cb}


class LiveBokehChart(object):
    """Base of the live charts: collects through ``pandas_logger`` and redraws at most every ``display_freq`` seconds."""

    def __init__(self, pandas_logger, metric_name, display_freq=10, batch_size=None, frequent=50):
        self.pandas_logger = pandas_logger or PandasLogger(batch_size=batch_size, frequent=frequent)
        self.display_freq = display_freq
        self.last_update = time.time()
        self.metric_name = metric_name
        self.handle = None
        self.fig = None
        if _bokeh_plotting is not None:
            _bokeh_io.output_notebook()
            self.handle = self.setup_chart()

    def setup_chart(self):
        raise NotImplementedError('an incomplete base class')

    def update_chart_data(self):
        raise NotImplementedError('an incomplete base class')

    def interval_elapsed(self):
        return time.time() - self.last_update > self.display_freq

    def _push_render(self):
        if _bokeh_io is not None and self.handle is not None:
            _bokeh_io.push_notebook(handle=self.handle)
        self.last_update = time.time()

    def _do_update(self):
        self.update_chart_data()
        self._push_render()

    def batch_cb(self, param):
        if self.interval_elapsed():
            self._do_update()

    def eval_cb(self, param):
        self._do_update()

    def callback_args(self):
        return {'batch_end_callback': self.batch_cb, 'eval_end_callback': self.eval_cb}


class LiveTimeSeries(LiveBokehChart):
    """A running value against the seconds since the chart was created."""

    def __init__(self, **fig_params):
        self.fig_params = fig_params
        self.start_time = datetime.datetime.now()
        self.x_axis_val, self.y_axis_val = [], []
        super().__init__(None, None, batch_size=1)

    def setup_chart(self):
        self.fig = _bokeh_plotting.figure(**self.fig_params)
        self._line = self.fig.line(self.x_axis_val, self.y_axis_val)
        return _bokeh_io.show(self.fig, notebook_handle=True)

    def elapsed(self):
        return (datetime.datetime.now() - self.start_time).total_seconds()

    def update_chart_data(self, value=None):
        if value is not None:
            self.x_axis_val.append(self.elapsed())
            self.y_axis_val.append(value)
        if self.fig is not None:
            self._line.data_source.data = {'x': list(self.x_axis_val), 'y': list(self.y_axis_val)}
        self._push_render()


class LiveLearningCurve(LiveBokehChart):
    """Training and validation values of one metric against the elapsed time."""

    def __init__(self, metric_name, display_freq=10, frequent=50):
        self.frequent = frequent
        self.start_time = datetime.datetime.now()
        self._data = {'train': {'elapsed': [], metric_name: []}, 'eval': {'elapsed': [], metric_name: []}}
        self._lines = {}
        super().__init__(None, metric_name, display_freq, batch_size=1, frequent=frequent)

    def setup_chart(self):
        self.fig = _bokeh_plotting.figure(x_axis_type='datetime', x_axis_label='Training time')
        for key, color in (('train', 'blue'), ('eval', 'red')):
            self._lines[key] = self.fig.line([], [], color=color, legend_label=key)
        return _bokeh_io.show(self.fig, notebook_handle=True)

    def _process(self, param, key):
        for name, value in _metric_pairs(param):
            if name == self.metric_name:
                self._data[key]['elapsed'].append(datetime.datetime.now() - self.start_time)
                self._data[key][self.metric_name].append(value)

    def batch_cb(self, param):
        if param.nbatch % self.frequent == 0:
            self._process(param, 'train')
        if self.interval_elapsed():
            self._do_update()

    def eval_cb(self, param):
        self._process(param, 'eval')
        self._do_update()

    def update_chart_data(self):
        for key, line in self._lines.items():
            line.data_source.data = {'x': list(self._data[key]['elapsed']), 'y': list(self._data[key][self.metric_name])}

    def _do_update(self):
        self.update_chart_data()
        self._push_render()


def args_wrapper(*args):
    """Merge the ``callback_args`` of several callback objects into one keyword dict (lists of callbacks)."""
    out = {}
    for a in args:
        for k, v in a.callback_args().items():
            out.setdefault(k, []).append(v)
    return out
