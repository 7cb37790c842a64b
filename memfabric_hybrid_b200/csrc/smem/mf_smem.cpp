// smem.h entry points: library init, stand-alone config-store servers, logging, TLS knobs, last error.
// Parity: src/smem/csrc/smem.cpp, src/smem/include/host/smem.h:55-182.
#include "../store/mf_store_backend.h"
#include "../util/mf_trace.h"
#include "mf_smem_common.h"

using namespace mf;

namespace mf {
namespace smem {
namespace {
std::atomic<int> g_inited{0};
}
bool SmemInited() { return g_inited.load() > 0; }
}  // namespace smem
}  // namespace mf

extern "C" {

int32_t smem_init(uint32_t flags)
{
    (void)flags;
    smem::g_inited.fetch_add(1);
    return SMEM_OK;
}

void smem_uninit(void)
{
    int v = smem::g_inited.load();
    while (v > 0 && !smem::g_inited.compare_exchange_weak(v, v - 1)) {}
    if (v == 1) store::StoreFactory::DestroyAll();
}

int32_t smem_create_config_store(const char *storeUrl, uint64_t flags)
{
    if (storeUrl == nullptr || *storeUrl == 0) return MF_FAIL(SMEM_INVALID_PARAM, "store url is empty");
    store::StoreUrl u;
    if (!store::StoreUrl::Parse(storeUrl, u)) return MF_FAIL(SMEM_INVALID_PARAM, "bad store url %s", storeUrl);
    if (u.scheme == store::StoreUrl::TCP) return smem::Pub(store::StoreFactory::CreateServerOnly(storeUrl, 0, flags));
    int err = OK;
    auto st = store::StoreFactory::CreateStore(storeUrl, true, 0, 0xFFFF0000u, 30000, flags, &err);
    return st ? SMEM_OK : smem::Pub(err);
}

void smem_destroy_config_store(const char *storeUrl)
{
    if (storeUrl == nullptr) return;
    store::StoreUrl u;
    if (store::StoreUrl::Parse(storeUrl, u) && u.scheme == store::StoreUrl::TCP) store::StoreFactory::DestroyServer(storeUrl);
    else store::StoreFactory::DestroyStore(storeUrl);
}

int32_t smem_config_store_set_backend_op(const smem_conf_store_backend_op_t *backendOp)
{
    return smem::Pub(store::SetExternalBackendOps(backendOp));
}

int32_t smem_set_extern_logger(void (*func)(int level, const char *msg))
{
    Logger::Get().SetSink(func);
    return SMEM_OK;
}

int32_t smem_set_extern_alarm(void (*alarm)(uint16_t code, const char *msg), void (*resume)(uint16_t code))
{
    Logger::Get().SetAlarm(alarm, resume);
    return SMEM_OK;
}

int32_t smem_set_log_level(int level)
{
    if (level < LOG_DEBUG || level > LOG_OFF) return MF_FAIL(SMEM_INVALID_PARAM, "log level %d out of [0,4]", level);
    Logger::Get().SetLevel(level);
    return SMEM_OK;
}

int32_t smem_set_conf_store_tls(bool enable, const char *tls_info, const uint32_t tls_info_len)
{
    if (enable && (tls_info == nullptr || tls_info_len == 0)) return MF_FAIL(SMEM_INVALID_PARAM, "TLS enabled without TLS info");
    return smem::Pub(store::StoreFactory::SetTls(enable, enable ? std::string(tls_info, tls_info_len) : std::string()));
}

int32_t smem_set_config_store_tls_key(const char *tls_pk, const uint32_t tls_pk_len, const char *tls_pk_pw,
                                      const uint32_t tls_pk_pw_len, const smem_decrypt_handler h)
{
    if (tls_pk == nullptr || tls_pk_len == 0) return smem::Pub(store::StoreFactory::SetTlsKey("", "", nullptr));  // forget the key
    // tls_pk: the key as PEM text, or the path of a PEM file. tls_pk_pw: its pass phrase (cipher text when a decrypt
    // handler is given). Takes effect for stores created after this call.
    std::string pass = (tls_pk_pw != nullptr && tls_pk_pw_len > 0) ? std::string(tls_pk_pw, tls_pk_pw_len) : std::string();
    return smem::Pub(store::StoreFactory::SetTlsKey(std::string(tls_pk, tls_pk_len), pass, h));
}

const char *smem_get_last_err_msg(void) { return LastError::Msg(); }
int32_t smem_get_last_err_code(void) { return LastError::Code(); }
const char *smem_get_and_clear_last_err_msg(void) { return LastError::TakeMsg(); }

}  // extern "C"
