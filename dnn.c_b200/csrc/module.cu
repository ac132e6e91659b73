// Module tree (parameter registration, flat parameter list, "DNNM" state
// files) and the thin layer structs.  Host-side glue only: the compute is in
// the ops these wrappers call.
// replaces src/module.c and src/nn.c of the reference.
#include "common.cuh"
#include <vector>
#include <string>
#include <functional>

using namespace dnnb;

namespace {

void append_item(module *m, module_item_kind kind, const char *name, tensor *param, module *child) {
    module_item *it = host_alloc_t<module_item>(m->pool);
    it->kind = kind; it->name = name;
    if (kind == MODULE_ITEM_PARAM) it->as.param = param; else it->as.child = child;
    if (m->items_tail) m->items_tail->next = it; else m->items_head = it;
    m->items_tail = it;
    m->n_items++;
}

void check_not_flattened(const module *m) {
    for (; m; m = m->parent)
        DNN_CHECK(m->flat_params == nullptr, "module: registration after module_parameters() was called");
}

// Depth-first walk in registration order; `path` is the dotted name.
void walk_params(module *m, std::string &path, const std::function<void(const std::string &, tensor *)> &f) {
    for (module_item *it = m->items_head; it; it = it->next) {
        size_t keep = path.size();
        path += it->name;
        if (it->kind == MODULE_ITEM_PARAM) f(path, it->as.param);
        else { path += '.'; walk_params(it->as.child, path, f); }
        path.resize(keep);
    }
}

void fill_ones(tensor *t) { k_fill((float *)t->data, numel_of(t), 1.0f); }

}  // namespace

extern "C" {

// ── module tree (src/module.c:60-165) ────────────────────────────────────
void module_init(module *m, struct mem_pool *pool, const char *type_name) {
    DNN_CHECK(m && pool && type_name, "module_init: NULL argument");
    memset(m, 0, sizeof *m);
    m->pool = pool; m->type_name = type_name;
}

void module_param(module *m, const char *name, tensor *t) {
    DNN_CHECK(m && name && t, "module_param: NULL argument");
    DNN_CHECK(t->pool == m->pool, "module_param: param must live in the module's params pool");
    DNN_CHECK(t->parent == nullptr && t->contiguous, "module_param: params must be contiguous non-views");
    check_not_flattened(m);
    append_item(m, MODULE_ITEM_PARAM, name, t, nullptr);
    m->n_direct_params++;
}

void module_add_child(module *m, const char *name, module *child) {
    DNN_CHECK(m && name && child && child != m, "module_add_child: bad argument");
    DNN_CHECK(child->pool == m->pool, "module_add_child: child must use the same params pool");
    DNN_CHECK(child->parent == nullptr, "module_add_child: child already has a parent");
    check_not_flattened(m);
    append_item(m, MODULE_ITEM_CHILD, name, nullptr, child);
    m->n_children++;
    child->parent = m;
}

tensor **module_parameters(module *m, int *n_out) {
    DNN_CHECK(m && n_out, "module_parameters: NULL argument");
    if (!m->flat_params) {
        std::vector<tensor *> flat;
        std::string path;
        walk_params(m, path, [&](const std::string &, tensor *t) {
            for (tensor *u : flat) if (u == t) return;       // shared (tied) params appear once
            flat.push_back(t);
        });
        m->flat_params = host_alloc_t<tensor *>(m->pool, flat.size() ? flat.size() : 1);
        for (size_t i = 0; i < flat.size(); i++) m->flat_params[i] = flat[i];
        m->n_flat = (int)flat.size();
    }
    *n_out = m->n_flat;
    return m->flat_params;
}

long long module_num_parameters(module *m) {
    int n; tensor **p = module_parameters(m, &n);
    long long total = 0;
    for (int i = 0; i < n; i++) total += numel_of(p[i]);
    return total;
}

void module_zero_grad(module *m) {
    int n; tensor **p = module_parameters(m, &n);
    for (int i = 0; i < n; i++) tensor_zero_grad(p[i]);
}

tensor *module_find_param(module *m, const char *name) {
    DNN_CHECK(m && name, "module_find_param: NULL argument");
    tensor *found = nullptr;
    std::string path;
    walk_params(m, path, [&](const std::string &p, tensor *t) { if (!found && p == name) found = t; });
    return found;
}

// ── state files (src/module.c:174-339; layout in include/module.h:94-98) ──
// magic "DNNM", u32 version=1, u32 header_size=16, u32 n_entries, then per
// entry: u32 name_len (with NUL), name, u32 ndim, i32 shape[ndim], u32 numel,
// float data[numel].  Weights only.  Payloads cross the PCIe bus here.
void module_save(module *m, const char *path) {
    DNN_CHECK(m && path, "module_save: NULL argument");
    FILE *f = fopen(path, "wb");
    DNN_CHECK(f, "module_save: cannot open file");
    uint32_t n_entries = 0;
    std::string p;
    walk_params(m, p, [&](const std::string &, tensor *) { n_entries++; });
    uint32_t version = 1, header = 16;
    fwrite("DNNM", 1, 4, f); fwrite(&version, 4, 1, f); fwrite(&header, 4, 1, f); fwrite(&n_entries, 4, 1, f);
    std::vector<float> host;
    walk_params(m, p, [&](const std::string &name, tensor *t) {
        uint32_t name_len = (uint32_t)name.size() + 1, ndim = (uint32_t)t->ndim, numel = (uint32_t)numel_of(t);
        fwrite(&name_len, 4, 1, f); fwrite(name.c_str(), 1, name_len, f); fwrite(&ndim, 4, 1, f);
        for (int d = 0; d < t->ndim; d++) { int32_t s = t->shape[d]; fwrite(&s, 4, 1, f); }
        fwrite(&numel, 4, 1, f);
        host.resize(numel);
        dnn_cuda_download(t, host.data(), (size_t)numel * 4);
        fwrite(host.data(), 4, numel, f);
    });
    fclose(f);
}

void module_load(module *m, const char *path, int strict) {
    DNN_CHECK(m && path, "module_load: NULL argument");
    FILE *f = fopen(path, "rb");
    DNN_CHECK(f, "module_load: cannot open file");
    char magic[4]; uint32_t version = 0, header = 0, n_entries = 0;
    DNN_CHECK(fread(magic, 1, 4, f) == 4 && memcmp(magic, "DNNM", 4) == 0, "module_load: bad magic");
    DNN_CHECK(fread(&version, 4, 1, f) == 1 && fread(&header, 4, 1, f) == 1 && fread(&n_entries, 4, 1, f) == 1,
              "module_load: truncated header");
    DNN_CHECK(version == 1 && header == 16, "module_load: unsupported version");
    std::vector<std::pair<std::string, tensor *>> live;
    std::string p;
    walk_params(m, p, [&](const std::string &name, tensor *t) { live.emplace_back(name, t); });
    std::vector<char> seen(live.size(), 0);
    std::vector<float> host;
    std::vector<char> name;
    for (uint32_t e = 0; e < n_entries; e++) {
        uint32_t name_len = 0, ndim = 0, numel = 0;
        int32_t shape[DNN_MAX_DIMS];
        DNN_CHECK(fread(&name_len, 4, 1, f) == 1 && name_len > 0 && name_len < MODULE_STATE_MAX_NAME, "module_load: bad name length");
        name.resize(name_len);
        DNN_CHECK(fread(name.data(), 1, name_len, f) == name_len && name[name_len - 1] == '\0', "module_load: truncated name");
        DNN_CHECK(fread(&ndim, 4, 1, f) == 1 && ndim > 0 && ndim <= DNN_MAX_DIMS, "module_load: bad ndim");
        DNN_CHECK(fread(shape, 4, ndim, f) == ndim, "module_load: truncated shape");
        DNN_CHECK(fread(&numel, 4, 1, f) == 1, "module_load: truncated entry");
        uint32_t prod = 1;
        for (uint32_t d = 0; d < ndim; d++) { DNN_CHECK(shape[d] > 0, "module_load: bad dim"); prod *= (uint32_t)shape[d]; }
        DNN_CHECK(prod == numel, "module_load: numel does not match shape");
        int idx = -1;
        for (size_t i = 0; i < live.size(); i++) if (live[i].first == name.data()) { idx = (int)i; break; }
        if (idx < 0) {
            DNN_CHECK(!strict, "module_load: unknown param in file");
            fseek(f, (long)numel * 4, SEEK_CUR);
            continue;
        }
        tensor *t = live[idx].second;
        DNN_CHECK((uint32_t)t->ndim == ndim, "module_load: ndim mismatch");
        for (uint32_t d = 0; d < ndim; d++) DNN_CHECK(t->shape[d] == shape[d], "module_load: shape mismatch");
        host.resize(numel);
        DNN_CHECK(fread(host.data(), 4, numel, f) == numel, "module_load: truncated data");
        dnn_cuda_upload(t, host.data(), (size_t)numel * 4);
        dnn_cuda_sync();        // `host` is reused by the next entry
        seen[idx] = 1;
    }
    if (strict) for (char s : seen) DNN_CHECK(s, "module_load: live param missing from file");
    fclose(f);
}

// ── layers (src/nn.c:10-199) ──────────────────────────────────────────────
linear *linear_create(struct mem_pool *params, int in_features, int out_features) {
    DNN_CHECK(in_features > 0 && out_features > 0, "linear_create: sizes must be positive");
    linear *l = host_alloc_t<linear>(params);
    module_init(&l->base, params, "linear");
    l->in_features = in_features; l->out_features = out_features;
    float bound = 1.0f / sqrtf((float)in_features);
    int ws[2] = {in_features, out_features}, bs[1] = {out_features};
    l->weight = tensor_uniform(params, 2, ws, 1, bound);
    l->bias = tensor_uniform(params, 1, bs, 1, bound);
    module_param(&l->base, "weight", l->weight);
    module_param(&l->base, "bias", l->bias);
    return l;
}
tensor *linear_forward(struct mem_pool *scratch, linear *l, const tensor *input) {
    DNN_CHECK(l && input && input->ndim >= 2, "linear_forward: input must be at least 2D");
    DNN_CHECK(input->shape[input->ndim - 1] == l->in_features, "linear_forward: last dim must match in_features");
    return tensor_matmul_add(scratch, input, l->weight, 0, l->bias);
}

swiglu_ffn *swiglu_ffn_create(struct mem_pool *params, int d_model, int intermediate_size) {
    DNN_CHECK(d_model > 0 && intermediate_size > 0, "swiglu_ffn_create: sizes must be positive");
    swiglu_ffn *ffn = host_alloc_t<swiglu_ffn>(params);
    module_init(&ffn->base, params, "swiglu_ffn");
    ffn->d_model = d_model; ffn->intermediate_size = intermediate_size;
    ffn->gate_proj = linear_create(params, d_model, intermediate_size);
    module_add_child(&ffn->base, "gate_proj", &ffn->gate_proj->base);
    ffn->up_proj = linear_create(params, d_model, intermediate_size);
    module_add_child(&ffn->base, "up_proj", &ffn->up_proj->base);
    ffn->down_proj = linear_create(params, intermediate_size, d_model);
    module_add_child(&ffn->base, "down_proj", &ffn->down_proj->base);
    return ffn;
}
tensor *swiglu_ffn_forward(struct mem_pool *scratch, swiglu_ffn *ffn, const tensor *x) {
    DNN_CHECK(ffn && x && x->ndim >= 2 && x->shape[x->ndim - 1] == ffn->d_model, "swiglu_ffn_forward: bad input");
    tensor *gate = linear_forward(scratch, ffn->gate_proj, x);
    tensor *up = linear_forward(scratch, ffn->up_proj, x);
    tensor *hidden = tensor_swiglu(scratch, gate, up);
    return linear_forward(scratch, ffn->down_proj, hidden);
}

layer_norm *layer_norm_create(struct mem_pool *params, int d, float eps) {
    DNN_CHECK(d > 0, "layer_norm_create: d must be positive");
    layer_norm *ln = host_alloc_t<layer_norm>(params);
    module_init(&ln->base, params, "layer_norm");
    ln->d = d; ln->eps = eps;
    ln->weight = tensor_zeros(params, 1, &d, 1);
    ln->bias = tensor_zeros(params, 1, &d, 1);
    fill_ones(ln->weight);
    module_param(&ln->base, "weight", ln->weight);
    module_param(&ln->base, "bias", ln->bias);
    return ln;
}
tensor *layer_norm_forward(struct mem_pool *scratch, layer_norm *ln, const tensor *x) {
    DNN_CHECK(ln && x, "layer_norm_forward: NULL argument");
    return tensor_layer_norm(scratch, x, ln->weight, ln->bias, ln->eps);
}

rms_norm *rms_norm_create(struct mem_pool *params, int d, float eps) {
    DNN_CHECK(d > 0, "rms_norm_create: d must be positive");
    rms_norm *rn = host_alloc_t<rms_norm>(params);
    module_init(&rn->base, params, "rms_norm");
    rn->d = d; rn->eps = eps;
    rn->weight = tensor_zeros(params, 1, &d, 1);
    fill_ones(rn->weight);
    module_param(&rn->base, "weight", rn->weight);
    return rn;
}
tensor *rms_norm_forward(struct mem_pool *scratch, rms_norm *rn, const tensor *x) {
    DNN_CHECK(rn && x, "rms_norm_forward: NULL argument");
    return tensor_rms_norm(scratch, x, rn->weight, rn->eps);
}

embedding *embedding_create(struct mem_pool *params, int vocab_size, int d_model) {
    DNN_CHECK(vocab_size > 0 && d_model > 0, "embedding_create: sizes must be positive");
    embedding *e = host_alloc_t<embedding>(params);
    module_init(&e->base, params, "embedding");
    e->vocab_size = vocab_size; e->d_model = d_model;
    int ws[2] = {vocab_size, d_model};
    e->weight = tensor_uniform(params, 2, ws, 1, 1.0f / sqrtf((float)d_model));
    module_param(&e->base, "weight", e->weight);
    return e;
}
tensor *embedding_forward(struct mem_pool *scratch, struct mem_pool *data, embedding *emb, const tensor *ids) {
    (void)data;
    DNN_CHECK(emb && ids, "embedding_forward: NULL argument");
    return tensor_embedding(scratch, emb->weight, ids);
}

conv2d *conv2d_create(struct mem_pool *params, int in_channels, int out_channels, int kernel_size, int stride, int padding) {
    DNN_CHECK(in_channels > 0 && out_channels > 0 && kernel_size > 0, "conv2d_create: sizes must be positive");
    conv2d *c = host_alloc_t<conv2d>(params);
    module_init(&c->base, params, "conv2d");
    c->in_channels = in_channels; c->out_channels = out_channels; c->kernel_size = kernel_size;
    c->stride = stride; c->padding = padding;
    float bound = sqrtf(6.0f / (float)(in_channels * kernel_size * kernel_size));
    int ws[4] = {out_channels, in_channels, kernel_size, kernel_size};
    c->weight = tensor_uniform(params, 4, ws, 1, bound);
    c->bias = tensor_zeros(params, 1, &out_channels, 1);
    module_param(&c->base, "weight", c->weight);
    module_param(&c->base, "bias", c->bias);
    return c;
}
tensor *conv2d_forward(struct mem_pool *scratch, conv2d *c, const tensor *input) {
    DNN_CHECK(c && input, "conv2d_forward: NULL argument");
    return tensor_conv2d(scratch, (tensor *)input, c->weight, c->bias, c->stride, c->padding);
}

}  // extern "C"
