// C ABI of the node-local rendezvous on its own (no GPU involved): used by the
// CPU test tier and by tools that only need the host-side exchange.
#include <unistd.h>
#include <cstring>
#include <string>
#include <vector>
#include "../api/oob.h"
#include "bootstrap.h"
#include "errors.h"

struct oob_bootstrap {
  oob::Bootstrap* b;
};

extern "C" {

int oob_bootstrap_create(int rank, int world, const char* key, int timeout_ms, oob_bootstrap** out) {
  if (out == nullptr || key == nullptr) return oob::set_error(OOB_ERR_INVALID, "null argument");
  std::string err;
  oob::Bootstrap* b = oob::Bootstrap::create(rank, world, key, timeout_ms, &err);
  if (b == nullptr) return oob::set_error(OOB_ERR_BOOTSTRAP, err);
  *out = new oob_bootstrap{b};
  return OOB_OK;
}

int oob_bootstrap_destroy(oob_bootstrap* h) {
  if (h != nullptr) {
    delete h->b;
    delete h;
  }
  return OOB_OK;
}

int oob_bootstrap_allgather(oob_bootstrap* h, const void* in, void* out, uint64_t bytes) {
  if (h == nullptr) return oob::set_error(OOB_ERR_INVALID, "null handle");
  if (!h->b->allgather(in, out, bytes)) return oob::set_error(OOB_ERR_BOOTSTRAP, h->b->last_error());
  return OOB_OK;
}

int oob_bootstrap_barrier(oob_bootstrap* h) {
  if (h == nullptr) return oob::set_error(OOB_ERR_INVALID, "null handle");
  if (!h->b->barrier()) return oob::set_error(OOB_ERR_BOOTSTRAP, h->b->last_error());
  return OOB_OK;
}

int oob_bootstrap_exchange_fds(oob_bootstrap* h, int my_fd, int* fds_out) {
  if (h == nullptr || fds_out == nullptr) return oob::set_error(OOB_ERR_INVALID, "null argument");
  std::vector<int> fds;
  if (!h->b->exchange_fds(my_fd, &fds)) return oob::set_error(OOB_ERR_BOOTSTRAP, h->b->last_error());
  for (size_t i = 0; i < fds.size(); ++i) fds_out[i] = fds[i];
  return OOB_OK;
}

int oob_bootstrap_broadcast_fd(oob_bootstrap* h, int root, int* fd) {
  if (h == nullptr || fd == nullptr) return oob::set_error(OOB_ERR_INVALID, "null argument");
  if (!h->b->broadcast_fd(root, fd)) return oob::set_error(OOB_ERR_BOOTSTRAP, h->b->last_error());
  return OOB_OK;
}

}  // extern "C"
